// tcgen05 implicit-GEMM convolution / GEMM for sm_100a.
//
// One kernel serves Conv, Gemm/MatMul (a 1x1 convolution over an [M, K] matrix), QLinearConv,
// QLinearMatMul, MatMulInteger and ConvInteger:
//
//   D[m, oc] = sum_{r,s,c} X[n, p*sh + r*dh - pt, q*sw + s*dw - pl, c] * Wp[oc, (r*S+s)*C + c]
//
// with m = (n*P + p)*Q + q over an NHWC activation tensor and K-major packed weights.
//
//  * A tiles (128 output pixels x one channel block of one filter tap) are gathered straight
//    from the NHWC activation by TMA in im2col mode (cp.async.bulk.tensor ... im2col), so no
//    im2col matrix ever exists in memory; plain GEMMs and 1x1/stride-1 convolutions use a 2-D
//    tiled TMA load of the same shape.  Padding taps arrive as zeros (TMA out-of-bounds fill).
//  * B tiles (BN output channels x the same K slice) are 2-D tiled TMA loads.
//  * No load uses cluster multicast: every CTA fetches its own tiles.
//  * One elected thread issues tcgen05.mma (kind::i8 with s32 accumulation, or kind::tf32 with
//    f32 accumulation) from shared-memory descriptors into one of two TMEM accumulators of BN
//    columns; a ring stage carries up to four K blocks when they are small, so that the
//    barrier round trip and the fixed cost of each asynchronous instruction are paid per stage.
//  * Eight epilogue warps (two per scheduler; the two of a TMEM lane quarter split the channel
//    runs) read the accumulator with tcgen05.ld (one output pixel per thread, 32 channels per
//    load), apply the fused epilogue in registers and hand the tile to TMA stores through
//    swizzled staging rows.  Epilogue variants, one tile loop instantiated per variant: float
//    bias / ReLU / clip / TF32 rounding, optionally with a fused residual; exact ONNX
//    requantisation in one fused multiply-add per output (and an f64 two-pass form for scales
//    outside its proven range); int32 saturation; the dequantising chain of a dynamically
//    quantised linear (scale, bias, Gelu).
//  * Batched products (attention) address each item's operands and output as windows of larger
//    row-major matrices, so heads are read and written in place.
//  * The grid is launched with programmatic stream serialization and waits for its predecessor
//    (griddepcontrol.wait) only after its own prologue.
//  * Every mbarrier wait is bounded; on a timeout the kernel records an error code, lets its
//    copies land, frees its TMEM and returns, so the context stays usable.
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "kernels.hpp"

namespace oxb {
namespace k {

namespace {

constexpr int BLOCK_M = 128;
// Eight epilogue warps, two per scheduler (one warp alone fills about half of its issue slots).
// Ten warps put three on two of the four schedulers, whose register files hold 16384 registers
// each: 168 registers per thread is the most this block shape can have.
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;  // warp 0: TMA producer, warp 1: MMA issuer + TMEM owner, warps 2-9: epilogue
constexpr int MAX_STAGES = 12;
constexpr long long WAIT_CYCLES = 2000000000LL;  // ~1 s at 2 GHz

struct alignas(64) KParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmO;
  int out_tma, out_row_bytes;
  int dbg;  // timing experiment only: 1 skips the epilogue work, 0 normal
  int a_im2col;
  int M, OC;
  int P, Q, S;
  int sh, sw, pt, pl, dh, dw;
  int taps, cblocks, cb_elems;
  int swizzle_bytes;  // 128, 64 or 32: bytes of K per shared-memory row (one K block)
  int kpb;            // K blocks per ring stage: one barrier round trip moves this many
  int stages;
  int n_tiles, m_tiles;
  // batched products (attention): tile t belongs to item t / (m_tiles * n_tiles) = (outer, inner); each operand
  // and the output start at row outer * rb + inner * rh and column inner * ch of their matrices
  int batched, items, items_inner;
  int a_rb, a_rh, a_ch, b_rb, b_rh, b_ch, o_rb, o_rh, o_ch;
  // split K (few output tiles, long K): work item t is (tile t / splits, slice t % splits); slice s runs K
  // blocks [s * k_per, (s + 1) * k_per) and leaves its raw accumulators in ws[tile][s][128 x BN]; per run of an
  // epilogue warp, the slice that arrives last (ws_count) adds the slices in order 0 .. splits-1 and runs the
  // fused epilogue.  Nobody waits for anybody, and the sum does not depend on the arrival order.  Counters are
  // kept per tile, epilogue warp and 32-channel run.
  int splits, k_per;
  uint32_t* ws;
  unsigned int* ws_count;
  uint32_t idesc;
  // epilogue
  int mode;
  int variant;  // which epilogue_math instantiation runs
  const float* bias_f;
  const float* residual;  // f32 [M, OC] added after the bias, or null
  int act;
  float clip_lo, clip_hi;
  int round_tf32;
  const int32_t* bias_i;
  const int32_t* wsum;
  const float* x_zp_dev;
  const float* combined;
  const float* dq_w_scale;   // dequantising epilogue: per-channel weight scale,
  const float* dq_x_scale;   // the activation's scale (one device lane),
  const float* dq_bias;      // per-channel f32 bias
  int y_zp, lo, hi;
  int out_dt;
  void* out;
  int* err_flag;
#ifdef OXB_UMMA_TRACE
  long long* trace;  // diagnostics build only: per-tile role timestamps of CTA 0
#endif
};

#ifdef OXB_UMMA_TRACE
#define OXB_TRACE(tile, slot)                                                             \
  do {                                                                                   \
    if (blockIdx.x == 0 && (tile) < 64 && lane == 0) p.trace[(tile) * 16 + (slot)] = clock64(); \
  } while (0)
#define OXB_TRACE_K(tile, it, slot)                                                                              \
  do {                                                                                                          \
    if (blockIdx.x == 0 && (tile) == 3 && (it) < 24 && lane == 0) p.trace[(40 + (it)) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define OXB_TRACE_K(tile, it, slot) \
  do {                              \
  } while (0)
#define OXB_TRACE(tile, slot) \
  do {                        \
  } while (0)
#endif

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: false when the barrier did not flip within WAIT_CYCLES or another role aborted.
// try_wait parks the warp in hardware for a bounded time per attempt, so a waiting role leaves
// its scheduler's issue slots to the epilogue warp that shares it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  long long start = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > WAIT_CYCLES) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
               "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h, int n, uint16_t off_w,
                                                    uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(
          dst),
      "l"((uint64_t)map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// The MMAs of one K block (1, 2 or 4 instructions of 32 bytes of K each) in one asm block: the
// 64-bit descriptors are assembled from a 32-bit low word that advances by 2 (16-byte units) per
// instruction and a constant high word, so the issuing thread spends a handful of integer
// instructions per K block.
#define OXB_MMA_BLOCK(KINDSTR)                                                                              \
  asm volatile(                                                                                             \
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"                                 \
      "setp.ne.b32 p, %5, 0;\n\tsetp.ne.b32 q, 1, 0;\n\t"                                                   \
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"                                                  \
      "tcgen05.mma.cta_group::1.kind::" KINDSTR " [%0], da, db, %4, p;\n\t"                                 \
      "setp.lt.u32 p, %6, 2;\n\t@p bra DONE_%=;\n\t"                                                        \
      "add.u32 la, %1, 2;\n\tadd.u32 lb, %2, 2;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::1.kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                                 \
      "setp.lt.u32 p, %6, 4;\n\t@p bra DONE_%=;\n\t"                                                        \
      "add.u32 la, %1, 4;\n\tadd.u32 lb, %2, 4;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::1.kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                                 \
      "add.u32 la, %1, 6;\n\tadd.u32 lb, %2, 6;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::1.kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                                 \
      "DONE_%=:\n\t}" ::"r"(tmem_d),                                                                        \
      "r"(lo_a), "r"(lo_b), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(mmas)                            \
      : "memory")

template <int KIND>
__device__ __forceinline__ void tc_mma_block(uint32_t tmem_d, uint32_t lo_a, uint32_t lo_b, uint32_t desc_hi, uint32_t idesc, uint32_t accumulate,
                                             uint32_t mmas) {
  if (KIND == 0) OXB_MMA_BLOCK("i8");
  else OXB_MMA_BLOCK("tf32");
}

// Shared-memory matrix descriptor, K-major operand, swizzled rows of `swz` bytes: start
// address, leading offset (unused for swizzled K-major, encoded 1), stride between 8-row
// groups (8 * swz bytes), descriptor version 1 (Blackwell), swizzle mode.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int swz) {
  uint64_t layout = swz == 128 ? 2ull : (swz == 64 ? 4ull : 6ull);
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(((uint32_t)(8 * swz) >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= layout << 61;
  return d;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// ---- the kernel ---------------------------------------------------------------------------
// Persistent: one CTA per SM walks the tile list (channel tile fastest, so CTAs that share an
// activation tile run together and meet in L2).  The shared-memory ring and the two TMEM
// accumulators are both pipelined across tiles: while the epilogue warps drain accumulator b,
// the MMA issuer fills accumulator b^1 and the producer is already loading further ahead.
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, naming the registers a pending read lands in: nothing that uses them may be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---- fused epilogue math ------------------------------------------------------------------
// One variant per (mode, activation, rounding) combination, chosen once per chunk, so that
// the 32 per-channel computations inside are straight-line code with full instruction-level
// parallelism (one epilogue warp per scheduler has nothing else to hide latency with).
// Per-channel parameters are read with 16-byte read-only loads; the host pads every
// parameter vector to a multiple of 256 channels, so no bounds checks are needed here.
enum { V_F32_BASE = 0, V_REQUANT = 6, V_REQUANT_DYN = 7, V_INT32 = 8, V_INT32_DYN = 9, V_REQUANT_FMA = 10, V_REQUANT_FMA_DYN = 11, V_REQUANT_LEAN = 12, V_REQUANT_LEAN_DYN = 13, V_F32_RES = 14,  // 14..19: the float variants with a residual
       V_DEQUANT = 20 };  // 20..25: dequantising variants, + (dynamic zero point ? 1 : 0) + 2 * activation

template <int ACT, int RT, bool RES>
__device__ __forceinline__ void math_f32(const KParams& p, const uint32_t (&v)[32], const float* __restrict__ bias, const float* __restrict__ res,
                                         uint32_t (&w)[32]) {
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const float4 b = __ldg(reinterpret_cast<const float4*>(bias) + j4);
    const float bb[4] = {b.x, b.y, b.z, b.w};
    float rr[4] = {0.f, 0.f, 0.f, 0.f};
    if (RES && res != nullptr) {  // this pixel's 32 channels of the residual: one full 128-byte line per thread
      const float4 r = __ldg(reinterpret_cast<const float4*>(res) + j4);
      rr[0] = r.x, rr[1] = r.y, rr[2] = r.z, rr[3] = r.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float f = __uint_as_float(v[4 * j4 + e]) + bb[e];
      if (RES) f = __fadd_rn(f, rr[e]);
      if (ACT == 1) f = fmaxf(f, 0.f);
      if (ACT == 2) f = fminf(fmaxf(f, p.clip_lo), p.clip_hi);
      if (RT) f = round_tf32(f);
      w[4 * j4 + e] = __float_as_uint(f);
    }
  }
}

// ONNX requantisation, bit-identical to the reference's
//   clamp(round_half_even(f64(acc) * f64(combined) + f64(zero_point)), lo, hi)
// without touching the (very narrow) FP64 pipe on the common path.  The value is formed in f32:
// a = (float)acc, r = fma(a, c, zp).  With |zp| <= 255, |r - exact| <= (2|r| + 255) * 2^-24 =: E.
// If r is further than T = (2|r| + 256) * 2^-23 >= 2E from every half-integer, the f32 value, the
// exact value and the reference's f64 value (within 2^-40 of exact) all round to the same integer.
// For |r| >= 1024 all three saturate on the same side.  Lanes within T of a tie (about one in ten
// thousand) are redone with the reference's own f64 operations in a second pass.
template <bool REQ, bool DYN>
__device__ __forceinline__ void math_int(const KParams& p, const uint32_t (&v)[32], const int32_t* __restrict__ bias, const int32_t* __restrict__ wsum,
                                         const float* __restrict__ comb, int xz, size_t esz, uint32_t (&w)[32]) {
  int32_t o[32];
  uint32_t slow = 0;
  const float zpf = (float)p.y_zp;
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const int4 b = __ldg(reinterpret_cast<const int4*>(bias) + j4);
    const int bb[4] = {b.x, b.y, b.z, b.w};
    int ss[4] = {0, 0, 0, 0};
    if (DYN) {
      const int4 sv = __ldg(reinterpret_cast<const int4*>(wsum) + j4);
      ss[0] = sv.x, ss[1] = sv.y, ss[2] = sv.z, ss[3] = sv.w;
    }
    float cc[4] = {0.f, 0.f, 0.f, 0.f};
    if (REQ) {
      const float4 c = __ldg(reinterpret_cast<const float4*>(comb) + j4);
      cc[0] = c.x, cc[1] = c.y, cc[2] = c.z, cc[3] = c.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int j = 4 * j4 + e;
      int32_t acc = (int32_t)v[j] + bb[e];
      if (DYN) acc -= xz * ss[e];
      if (REQ) {
        const float r = fmaf(__int2float_rn(acc), cc[e], zpf);
        const float q = rintf(r);
        const float t = fmaf(fabsf(r), 2.384185791015625e-07f, 3.0517578125e-05f);  // |r| * 2^-22 + 2^-15
        const bool near_tie = (fabsf(r - q) > 0.5f - t) && (fabsf(r) < 1024.0f);
        slow |= (near_tie ? 1u : 0u) << j;
        acc = min(max(__float2int_rn(r), p.lo), p.hi);
      }
      o[j] = acc;
    }
  }
  if (REQ && slow != 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if ((slow >> j) & 1u) {
        int32_t acc = (int32_t)v[j] + __ldg(bias + j);
        if (DYN) acc -= xz * __ldg(wsum + j);
        // f64 product and f64 add, each rounded once; round-half-even; saturate
        const double scaled = __dadd_rn(__dmul_rn((double)acc, (double)__ldg(comb + j)), (double)p.y_zp);
        o[j] = min(max(__double2int_rn(scaled), p.lo), p.hi);
      }
    }
  }
  if (esz == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j] = ((uint32_t)o[4 * j] & 0xffu) | (((uint32_t)o[4 * j + 1] & 0xffu) << 8) | (((uint32_t)o[4 * j + 2] & 0xffu) << 16) |
             (((uint32_t)o[4 * j + 3] & 0xffu) << 24);
  } else if (esz == 2) {
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = ((uint32_t)o[2 * j] & 0xffffu) | (((uint32_t)o[2 * j + 1] & 0xffffu) << 16);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = (uint32_t)o[j];
  }
}

// ONNX requantisation in one fused multiply-add per output.  With a = (float)acc exact
// (|acc| < 2^24) the instruction s = fma(a, c, 1.5 * 2^23 + zp) rounds the exact real number
// acc * c + zp once, to the integer grid of the binade [2^23, 2^24), ties to even: the low
// mantissa bits of s are round_half_even(acc * c + zp).  The reference's two f64 operations
// are exact for these operands (a 24-bit by 24-bit product, and a sum spanning at most 53
// bits when |c| >= 2^-21, which the host checks before choosing this variant), so both sides
// round the same real number the same way.  Values beyond +-2^22 leave the binade but stay
// monotone, and the clamp (done on the float, before the bits are taken) sends them to the
// same bound as the reference's.  A thread that meets |acc| >= 2^24 redoes those eight channels
// with the reference's own f64 operations; when the host can bound every accumulator of the layer
// below 2^24 from the weights, the variant without that check and second pass is used.
template <bool DYN, bool FALLBACK>
__device__ __forceinline__ void math_requant_fma(const KParams& p, const uint32_t (&v)[32], const int32_t* __restrict__ bias,
                                                 const int32_t* __restrict__ wsum, const float* __restrict__ comb, int xz, size_t esz,
                                                 uint32_t (&w)[32]) {
  const float magic = 12582912.0f;  // 1.5 * 2^23
  const float magic_zp = magic + (float)p.y_zp, flo = magic + (float)p.lo, fhi = magic + (float)p.hi;
  // eight channels at a time, packed at once: few values are live together, so that two runs can
  // be in flight per warp (one in TMEM transit) inside the register budget of a ten-warp block
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float amax = 0.f;
    uint32_t sb[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j4 = 2 * g + h;
      const int4 b = __ldg(reinterpret_cast<const int4*>(bias) + j4);
      const int bb[4] = {b.x, b.y, b.z, b.w};
      int ss[4] = {0, 0, 0, 0};
      if (DYN) {
        const int4 sv = __ldg(reinterpret_cast<const int4*>(wsum) + j4);
        ss[0] = sv.x, ss[1] = sv.y, ss[2] = sv.z, ss[3] = sv.w;
      }
      const float4 c = __ldg(reinterpret_cast<const float4*>(comb) + j4);
      const float cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int32_t acc = (int32_t)v[4 * j4 + e] + bb[e];
        if (DYN) acc -= xz * ss[e];
        const float a = __int2float_rn(acc);
        if (FALLBACK) amax = fmaxf(amax, fabsf(a));
        sb[4 * h + e] = __float_as_uint(fminf(fmaxf(fmaf(a, cc[e], magic_zp), flo), fhi));
      }
    }
    // the value sits in the low mantissa bits (two's complement below 2^22): take its low byte,
    // or its low half-word for the 16-bit lanes of the union range [-128, 255]
    if (esz == 1) {
      w[2 * g] = __byte_perm(__byte_perm(sb[0], sb[1], 0x0040), __byte_perm(sb[2], sb[3], 0x0040), 0x5410);
      w[2 * g + 1] = __byte_perm(__byte_perm(sb[4], sb[5], 0x0040), __byte_perm(sb[6], sb[7], 0x0040), 0x5410);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) w[4 * g + k] = __byte_perm(sb[2 * k], sb[2 * k + 1], 0x5410);
    }
    if (FALLBACK && amax >= 16777216.0f) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int j = 8 * g + k;
        int32_t acc = (int32_t)v[j] + __ldg(bias + j);
        if (DYN) acc -= xz * __ldg(wsum + j);
        const double scaled = __dadd_rn(__dmul_rn((double)acc, (double)__ldg(comb + j)), (double)p.y_zp);
        const uint32_t q = (uint32_t)min(max(__double2int_rn(scaled), p.lo), p.hi);
        if (esz == 1) w[j >> 2] = (w[j >> 2] & ~(0xffu << (8 * (j & 3)))) | ((q & 0xffu) << (8 * (j & 3)));
        else w[j >> 1] = (w[j >> 1] & ~(0xffffu << (16 * (j & 1)))) | ((q & 0xffffu) << (16 * (j & 1)));
      }
    }
  }
}

// erf by the reference's polynomial (Abramowitz-Stegun 7.1.26, nn_ops/activations.rs:578), same operation order.
__device__ __forceinline__ float erf_poly(float x) {
  const float sign = x >= 0.0f ? 1.0f : -1.0f;
  x = fabsf(x);
  const float t = __frcp_rn(__fadd_rn(1.0f, __fmul_rn(0.3275911f, x)));  // the correctly rounded 1 / d, as the division gives
  float p = __fadd_rn(-1.4531521f, __fmul_rn(t, 1.0614054f));
  p = __fadd_rn(1.4214138f, __fmul_rn(t, p));
  p = __fadd_rn(-0.28449672f, __fmul_rn(t, p));
  p = __fadd_rn(0.2548296f, __fmul_rn(t, p));
  return __fmul_rn(sign, __fsub_rn(1.0f, __fmul_rn(__fmul_rn(t, p), expf(__fmul_rn(-x, x)))));
}

// Dequantising epilogue of a dynamically quantised linear: the integer accumulator becomes an f32 lane
// (round to nearest even above 2^24, as `saturate_i32(acc) as f32`), is multiplied by x_scale * w_scale[oc]
// and gets bias[oc] added, each operation rounded on its own, then optionally Gelu.
template <bool DYN, int ACT>
__device__ __forceinline__ void math_dequant(const KParams& p, const uint32_t (&v)[32], const int32_t* __restrict__ bias_i,
                                             const int32_t* __restrict__ wsum, const float* __restrict__ wscale, const float* __restrict__ bias_f, int xz,
                                             float xs, uint32_t (&w)[32]) {
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const int4 b = __ldg(reinterpret_cast<const int4*>(bias_i) + j4);
    const int bb[4] = {b.x, b.y, b.z, b.w};
    int ss[4] = {0, 0, 0, 0};
    if (DYN) {
      const int4 sv = __ldg(reinterpret_cast<const int4*>(wsum) + j4);
      ss[0] = sv.x, ss[1] = sv.y, ss[2] = sv.z, ss[3] = sv.w;
    }
    const float4 c = __ldg(reinterpret_cast<const float4*>(wscale) + j4);
    const float cc[4] = {c.x, c.y, c.z, c.w};
    const float4 f = __ldg(reinterpret_cast<const float4*>(bias_f) + j4);
    const float ff[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int32_t acc = (int32_t)v[4 * j4 + e] + bb[e];
      if (DYN) acc -= xz * ss[e];
      float y = __fadd_rn(__fmul_rn(__int2float_rn(acc), __fmul_rn(xs, cc[e])), ff[e]);
      if (ACT == 1) y = __fmul_rn(__fmul_rn(y, 0.5f), __fadd_rn(1.0f, erf_poly(__fmul_rn(y, 0.70710678118654752440f))));
      if (ACT == 2) {
        const float inner = __fmul_rn(0.7978846f, __fadd_rn(y, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, y), y), y)));
        y = __fmul_rn(__fmul_rn(0.5f, y), __fadd_rn(1.0f, tanhf(inner)));
      }
      if (p.round_tf32) y = round_tf32(y);  // the lane feeds a TF32 product
      w[4 * j4 + e] = __float_as_uint(y);
    }
  }
}

// Fused epilogue of one 32-channel run of one output pixel: bias / zero-point correction,
// requantisation or activation, packed into 32-bit words (8 for 8-bit outputs, 16 for 16-bit,
// 32 for 32-bit).  `oc` is the first channel of the run.  The variant is a template argument:
// the whole tile loop of an epilogue warp is instantiated per variant, so the code a warp runs
// is one straight body without a dispatch inside the loop.
template <int VARIANT>
__device__ __forceinline__ void epilogue_chunk(const KParams& p, const uint32_t (&v)[32], int xz, int oc, size_t esz, const float* res, uint32_t (&w)[32]) {
  if constexpr (VARIANT < V_REQUANT) math_f32<VARIANT / 2, VARIANT & 1, false>(p, v, p.bias_f + oc, nullptr, w);
  else if constexpr (VARIANT >= V_DEQUANT) {
    const float xs = __ldg(p.dq_x_scale);
    math_dequant<((VARIANT - V_DEQUANT) & 1) != 0, (VARIANT - V_DEQUANT) / 2>(p, v, p.bias_i + oc, p.wsum + oc, p.dq_w_scale + oc, p.dq_bias + oc, xz, xs, w);
  } else if constexpr (VARIANT >= V_F32_RES) math_f32<(VARIANT - V_F32_RES) / 2, (VARIANT - V_F32_RES) & 1, true>(p, v, p.bias_f + oc, res, w);
  else if constexpr (VARIANT == V_REQUANT) math_int<true, false>(p, v, p.bias_i + oc, nullptr, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_DYN) math_int<true, true>(p, v, p.bias_i + oc, p.wsum + oc, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_INT32) math_int<false, false>(p, v, p.bias_i + oc, nullptr, nullptr, xz, esz, w);
  else if constexpr (VARIANT == V_INT32_DYN) math_int<false, true>(p, v, p.bias_i + oc, p.wsum + oc, nullptr, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_FMA) math_requant_fma<false, true>(p, v, p.bias_i + oc, nullptr, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_FMA_DYN) math_requant_fma<true, true>(p, v, p.bias_i + oc, p.wsum + oc, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_LEAN) math_requant_fma<false, false>(p, v, p.bias_i + oc, nullptr, p.combined + oc, xz, esz, w);
  else math_requant_fma<true, false>(p, v, p.bias_i + oc, p.wsum + oc, p.combined + oc, xz, esz, w);
}

// Direct store of a packed 32-channel run (ragged channel counts, unaligned rows).
__device__ __forceinline__ void store_direct(const uint32_t (&w)[32], uint8_t* optr, size_t esz, int valid) {
  const int bytes = 32 * (int)esz;
  if (valid == 32 && ((uintptr_t)optr & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j * 16 < bytes) *(uint4*)(optr + j * 16) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    return;
  }
  if (esz == 4) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) ((uint32_t*)optr)[j] = w[j];
  } else if (esz == 2) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) ((uint16_t*)optr)[j] = (uint16_t)(w[j >> 1] >> (16 * (j & 1)));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) optr[j] = (uint8_t)(w[j >> 2] >> (8 * (j & 3)));
  }
}

// Staged store: the run goes into this warp's shared-memory staging rows in the swizzled order a
// TMA store with the matching swizzle mode expects (16-byte chunk index XOR row-derived bits), so
// that the tile leaves the SM as full-line writes instead of 32 scattered 16-byte pieces.
__device__ __forceinline__ void store_staged(const uint32_t (&w)[32], uint32_t stage_addr, int row, int pitch, int byte_off, int bytes) {
  const uint32_t xor_bits = ((uint32_t)(row * pitch) >> 7) & (uint32_t)(pitch / 16 - 1);
  const uint32_t row_addr = stage_addr + (uint32_t)(row * pitch);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j * 16 < bytes) {
      const uint32_t chunk = ((uint32_t)(byte_off >> 4) + (uint32_t)j) ^ xor_bits;
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + chunk * 16u), "r"(w[4 * j]), "r"(w[4 * j + 1]), "r"(w[4 * j + 2]),
                   "r"(w[4 * j + 3])
                   : "memory");
    }
  }
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((uint64_t)map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}

// ---- epilogue role ------------------------------------------------------------------------
// Eight warps drain an accumulator: warp w may read the TMEM lanes 32 * (w % 4) .. + 31 (output
// rows of the tile), and the two warps of a lane quarter split the tile's channel runs in two
// contiguous halves.  Per run: TMEM read of the following run in flight, fused math, then
// either a swizzled copy into this warp's 4 KB staging rows followed by one TMA store per
// `pitch` bytes of row, or direct 16-byte stores.  The accumulator is handed back to the MMA
// issuer as soon as this warp's last TMEM read has landed, before the last run's math.
template <int BN, int VARIANT, bool SPLIT>
__device__ __forceinline__ void epilogue_role(const KParams& p, int warp, int lane, uint32_t tmem_base, uint64_t* bar_acc_full,
                                              uint64_t* bar_acc_empty, uint32_t stage_addr, volatile int* abortp, int total_tiles) {
  constexpr int CPW = BN >= 64 ? BN / 64 : 1;  // channel runs per warp and tile
  const int quarter = warp & 3;
  const int ew = warp - 2;
  const int first = (ew >> 2) * CPW;
  int xz = 0;
  if (p.x_zp_dev) xz = __float2int_rn(*p.x_zp_dev);
  const size_t esz = (p.out_dt == (int)DT::F32 || p.out_dt == (int)DT::I32) ? 4 : (p.out_dt == (int)DT::I16 ? 2 : 1);
  const int chunk_bytes = 32 * (int)esz;
  const int pitch = p.out_row_bytes;  // staged row length: 32, 64 or 128 bytes, at most one warp's share of a row
  const int cpg = p.out_tma ? pitch / chunk_bytes : 1;
  uint32_t local = 0;
  for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
    int tt = t, o_row0 = 0, o_col0 = 0;
    if (p.batched) {
      const int per = p.m_tiles * p.n_tiles, item = t / per;
      tt = t - item * per;
      const int outer = item / p.items_inner, inner = item - outer * p.items_inner;
      o_row0 = outer * p.o_rb + inner * p.o_rh;
      o_col0 = inner * p.o_ch;
    } else if (p.splits > 1) {
      tt = t / p.splits;
    }
    const int tile_n = tt % p.n_tiles, tile_m = tt / p.n_tiles;
    const int m0 = tile_m * BLOCK_M, oc0 = tile_n * BN;
    const uint32_t buf = local & 1u;
    if (ew == 0) OXB_TRACE(local, 6);
    bool ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (local >> 1) & 1u, abortp);
    if (ew == 0) OXB_TRACE(local, 7);
    if (!ok && !*abortp) {
      *abortp = 1;
      atomicExch(p.err_flag, 3);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    tc_fence_after();
    const long long m = (long long)m0 + quarter * 32 + lane;
    const bool row_ok = m < p.M;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)BN;
    const int n_chunks = min(BN, p.OC - oc0 + 31) / 32;  // uniform across the CTA
    const int end = min(first + CPW, n_chunks);           // this warp's runs: [first, end)
    uint32_t va[32], w[32];

    auto release = [&]() {  // every TMEM read of this warp for this tile has landed
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
    };
    auto math = [&](const uint32_t(&v)[32], int ch) {
      const float* res = (VARIANT >= V_F32_RES && VARIANT < V_DEQUANT && row_ok) ? p.residual + (size_t)m * p.OC + oc0 + ch * 32 : nullptr;
      epilogue_chunk<VARIANT>(p, v, xz, oc0 + ch * 32, esz, res, w);
    };
    auto store = [&](int ch) {
      if (p.out_tma) {
        const int in_group = (ch - first) % cpg;
        if (in_group == 0) {
          // the staging rows are rewritten: their previous store must have read them
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        }
        store_staged(w, stage_addr, lane, pitch, in_group * chunk_bytes, chunk_bytes);
        if (in_group == cpg - 1 || ch == end - 1) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&p.tmO, stage_addr, o_col0 + oc0 + (ch - in_group) * 32, o_row0 + m0 + quarter * 32);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else if (row_ok) {
        store_direct(w, (uint8_t*)p.out + ((size_t)m * p.OC + oc0 + ch * 32) * esz, esz, min(32, p.OC - (oc0 + ch * 32)));
      }
    };
    auto emit = [&](const uint32_t(&v)[32], int ch) {
      math(v, ch);
      store(ch);
    };

    if (p.dbg == 1 || first >= end) {  // timing experiment without epilogue work, or no run of this tile is ours
      release();
      continue;
    }
    if constexpr (SPLIT) {
      // Runs are taken in an order rotated by the slice index and each run has its own arrival counter, so the
      // slices of a tile finish different runs last and share the summing and the fused epilogue between them.
      constexpr bool kFloatAcc = VARIANT < V_REQUANT || (VARIANT >= V_F32_RES && VARIANT < V_DEQUANT);
      const int split = t - tt * p.splits;
      // workspace of one slice: [lane quarter][run][16-byte piece j][lane], so that every store and load of a
      // warp covers 512 contiguous bytes (only warps with the same index in the other slices read it back)
      const uint4* tile_ws = reinterpret_cast<const uint4*>(p.ws + (size_t)tt * p.splits * (BLOCK_M * BN)) + (size_t)quarter * (BN / 32) * 256 + lane;
      constexpr size_t kSlice = (size_t)BLOCK_M * BN / 4;  // 16-byte pieces per slice
      uint4* mine = const_cast<uint4*>(tile_ws) + (size_t)split * kSlice;
      unsigned int* counters = p.ws_count + ((size_t)tt * EPI_WARPS + ew) * 4;
      const int runs = end - first;
      for (int i = 0; i < runs; ++i) {
        const int c = first + (i + split) % runs;
        tmem_ld32_nowait(taddr + (uint32_t)c * 32u, va);
        tmem_ld_wait();
        if (i == runs - 1) release();
#pragma unroll
        for (int j = 0; j < 8; ++j) __stcg(mine + (c * 8 + j) * 32, make_uint4(va[4 * j], va[4 * j + 1], va[4 * j + 2], va[4 * j + 3]));
        __threadfence();
        __syncwarp();
        unsigned int arrived = 0;
        if (lane == 0) arrived = atomicAdd(counters + (c - first), 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != (unsigned int)p.splits - 1u) continue;  // a later slice finishes this run
        if (lane == 0) counters[c - first] = 0u;               // ready for the next launch
        __threadfence();
        for (int sl = 0; sl < p.splits; ++sl) {
          const uint4* src = tile_ws + (size_t)sl * kSlice + c * 256;
          uint4 xv[8];  // the eight loads of a slice are issued together
#pragma unroll
          for (int j = 0; j < 8; ++j) xv[j] = __ldcg(src + j * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t xs[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (sl == 0) va[4 * j + e] = xs[e];
              else if (kFloatAcc) va[4 * j + e] = __float_as_uint(__fadd_rn(__uint_as_float(va[4 * j + e]), __uint_as_float(xs[e])));
              else va[4 * j + e] += xs[e];
            }
          }
        }
        emit(va, c);
      }
      if (ew == 0) OXB_TRACE(local, 8);
      continue;
    }
    if constexpr (SPLIT) continue;  // (not reached)
    tmem_ld32_nowait(taddr + (uint32_t)first * 32u, va);
    tmem_ld_wait_for(va);
    // one copy of the run's code in the loop (the instruction cache is what this loop is short of); a run's math
    // leaves its packed words in `w`, so the next run's TMEM read can land in the same registers while the words
    // are staged and handed to the TMA store (no second register set, no copies between the two)
#pragma unroll 1
    for (int c = first; c < end; ++c) {
      const bool more = c + 1 < end;
      math(va, c);
      if (more) tmem_ld32_nowait(taddr + (uint32_t)(c + 1) * 32u, va);
      else release();
      store(c);
      if (more) tmem_ld_wait_for(va);
    }
    if (ew == 0) OXB_TRACE(local, 8);
    if (ew == EPI_WARPS - 1) OXB_TRACE(local, 9);
  }
  if (p.out_tma && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}


template <int BN, int KIND>
__global__ void __launch_bounds__(NUM_THREADS, 1) umma_conv_kernel(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  // per epilogue warp: staging rows (32 x up to 128 bytes) for the TMA stores
  __shared__ __align__(1024) uint8_t s_stage[EPI_WARPS][32 * 128];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int swz = p.swizzle_bytes;
  const uint32_t a_bytes = (uint32_t)BLOCK_M * swz, b_bytes = (uint32_t)BN * swz;
  const uint32_t kb_bytes = a_bytes + b_bytes;           // one K block: activations, then weights
  const uint32_t stage_bytes = kb_bytes * (uint32_t)p.kpb;  // one ring stage
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int k_iters = p.taps * p.cblocks;
  const int total_tiles = p.m_tiles * p.n_tiles * (p.batched ? p.items : p.splits);
  constexpr uint32_t TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bar_acc_full[i]), 1);
      mbar_init(smem_u32(&bar_acc_empty[i]), EPI_WARPS);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  // let the next grid in the stream start its own prologue, then wait for the previous grid's results
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // The producer and the MMA issuer run their loops with the whole warp (every lane polls the
  // barrier, one lane issues): a lone lane looping while its 31 siblings sit at the teardown
  // barrier gets only a fraction of the warp's issue slots.
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    uint32_t stage = 0, phase = 0;  // ring position, carried across tiles
    bool ok = true;
    int ptile = 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++ptile) {
      OXB_TRACE(ptile, 0);
      int tt = t, a_row0 = 0, a_col0 = 0, b_row0 = 0, b_col0 = 0;
      int it_begin = 0, it_end = k_iters;
      if (p.batched) {
        const int per = p.m_tiles * p.n_tiles, item = t / per;
        tt = t - item * per;
        const int outer = item / p.items_inner, inner = item - outer * p.items_inner;
        a_row0 = outer * p.a_rb + inner * p.a_rh;
        a_col0 = inner * p.a_ch;
        b_row0 = outer * p.b_rb + inner * p.b_rh;
        b_col0 = inner * p.b_ch;
      } else if (p.splits > 1) {
        tt = t / p.splits;
        it_begin = (t - tt * p.splits) * p.k_per;
        it_end = min(k_iters, it_begin + p.k_per);
      }
      const int tile_n = tt % p.n_tiles, tile_m = tt / p.n_tiles;
      const int m0 = tile_m * BLOCK_M, oc0 = tile_n * BN;
      int q0 = 0, p0 = 0, n0 = 0;
      if (p.a_im2col) {
        q0 = m0 % p.Q;
        int tt = m0 / p.Q;
        p0 = tt % p.P;
        n0 = tt / p.P;
      }
      const int w_base = q0 * p.sw - p.pl, h_base = p0 * p.sh - p.pt;
      int cb = it_begin % p.cblocks, sx = (it_begin / p.cblocks) % p.S, r = (it_begin / p.cblocks) / p.S;
      // A barrier round trip, an expect_tx and each TMA instruction cost the issuing thread on the
      // order of a hundred cycles, whatever the box size: a stage carries several K blocks when
      // they are small, so that those costs are paid once per stage.
      for (int it = it_begin; it < it_end; it += p.kpb) {
        OXB_TRACE_K(ptile, it, 0);
        bool got = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp);
        OXB_TRACE_K(ptile, it, 1);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*abortp) {
            *abortp = 1;
            atomicExch(p.err_flag, 1);
          }
          ok = false;
          break;
        }
        if (p.kpb == 1) {
          if (lane == 0) {  // one thread issues: every operand of the copies is warp-uniform
            const uint32_t full = smem_u32(&bar_full[stage]);
            mbar_expect_tx(full, kb_bytes);
            const uint32_t a_dst = tiles_base + stage * stage_bytes;
            const int c_off = cb * p.cb_elems;
            if (p.a_im2col) tma_load_im2col_4d(a_dst, &p.tmA, full, c_off, w_base, h_base, n0, (uint16_t)(sx * p.dw), (uint16_t)(r * p.dh));
            else tma_load_2d(a_dst, &p.tmA, full, a_col0 + c_off, a_row0 + m0);
            tma_load_2d(a_dst + a_bytes, &p.tmB, full, b_col0 + it * p.cb_elems, b_row0 + oc0);
          }
          if (++cb == p.cblocks) {
            cb = 0;
            if (++sx == p.S) {
              sx = 0;
              ++r;
            }
          }
        } else {
          const int blocks = min(p.kpb, it_end - it);
          const uint32_t full = smem_u32(&bar_full[stage]);
          if (lane == 0) mbar_expect_tx(full, kb_bytes * (uint32_t)blocks);
          uint32_t a_dst = tiles_base + stage * stage_bytes;
          for (int g = 0; g < blocks; ++g, a_dst += kb_bytes) {
            if (lane == 0) {
              const int c_off = cb * p.cb_elems;
              if (p.a_im2col) tma_load_im2col_4d(a_dst, &p.tmA, full, c_off, w_base, h_base, n0, (uint16_t)(sx * p.dw), (uint16_t)(r * p.dh));
              else tma_load_2d(a_dst, &p.tmA, full, a_col0 + c_off, a_row0 + m0);
              tma_load_2d(a_dst + a_bytes, &p.tmB, full, b_col0 + (it + g) * p.cb_elems, b_row0 + oc0);
            }
            if (++cb == p.cblocks) {
              cb = 0;
              if (++sx == p.S) {
                sx = 0;
                ++r;
              }
            }
          }
        }
        OXB_TRACE_K(ptile, it, 2);
        __syncwarp();
        if (++stage == (uint32_t)p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      OXB_TRACE(ptile, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t mmas = (uint32_t)(swz / 32);
    const uint64_t desc_rest = make_smem_desc(0, swz);
    const uint32_t desc_hi = (uint32_t)(desc_rest >> 32), desc_lo = (uint32_t)desc_rest;
    const uint32_t idesc = p.idesc;
    const uint32_t ring16 = tiles_base >> 4, stage16 = stage_bytes >> 4, kb16 = kb_bytes >> 4, a16_bytes = a_bytes >> 4;
    uint32_t stage = 0, phase = 0, a16 = ring16;
    uint32_t local = 0;
    bool ok = true;
    const bool one_block = p.kpb == 1;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      const uint32_t buf = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      OXB_TRACE(local, 2);
      // the epilogue must have drained this accumulator (free on the first two tiles)
      bool got = mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_phase ^ 1u, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0 && !*abortp) {
          *abortp = 1;
          atomicExch(p.err_flag, 4);
        }
        break;
      }
      tc_fence_after();
      OXB_TRACE(local, 3);
      const uint32_t tmem_d = tmem_base + buf * (uint32_t)BN;
      int it_begin = 0, it_end = k_iters;
      if (!p.batched && p.splits > 1) {
        it_begin = (t % p.splits) * p.k_per;
        it_end = min(k_iters, it_begin + p.k_per);
      }
      for (int it = it_begin; it < it_end; it += p.kpb) {
        OXB_TRACE_K((int)local, it, 3);
        got = mbar_wait(smem_u32(&bar_full[stage]), phase, abortp);
        OXB_TRACE_K((int)local, it, 4);
        if (it == it_begin) OXB_TRACE(local, 4);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*abortp) {
            *abortp = 1;
            atomicExch(p.err_flag, 2);
          }
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          // descriptors differ between K blocks only in the 16-byte granular start address
          if (one_block) {
            tc_mma_block<KIND>(tmem_d, desc_lo | (a16 & 0x3fffu), desc_lo | ((a16 + a16_bytes) & 0x3fffu), desc_hi, idesc, it > it_begin ? 1u : 0u, mmas);
          } else {
            const int blocks = min(p.kpb, it_end - it);
            uint32_t b16 = a16;
            for (int g = 0; g < blocks; ++g, b16 += kb16)
              tc_mma_block<KIND>(tmem_d, desc_lo | (b16 & 0x3fffu), desc_lo | ((b16 + a16_bytes) & 0x3fffu), desc_hi, idesc, (it + g) > it_begin ? 1u : 0u, mmas);
          }
          tc_commit(smem_u32(&bar_empty[stage]));  // frees the stage once these MMAs have read it
        }
        OXB_TRACE_K((int)local, it, 5);
        __syncwarp();
        a16 += stage16;
        if (++stage == (uint32_t)p.stages) {
          stage = 0;
          phase ^= 1u;
          a16 = ring16;
        }
      }
      if (ok && lane == 0) tc_commit(smem_u32(&bar_acc_full[buf]));  // accumulator complete
      __syncwarp();
      OXB_TRACE(local, 5);
    }
  } else {
    // ---------------- epilogue: warps 2..9 ----------------
    const uint32_t stage_addr = smem_u32(&s_stage[warp - 2][0]);
    const bool split = !p.batched && p.splits > 1;
#define OXB_EPI(V)                                                                                                                  \
  case V:                                                                                                                           \
    if (split) epilogue_role<BN, V, true>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);   \
    else epilogue_role<BN, V, false>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);        \
    break;
    if constexpr (KIND == 0) {
      switch (p.variant) {
        OXB_EPI(V_REQUANT)
        OXB_EPI(V_REQUANT_DYN)
        OXB_EPI(V_INT32)
        OXB_EPI(V_INT32_DYN)
        OXB_EPI(V_REQUANT_FMA)
        OXB_EPI(V_REQUANT_FMA_DYN)
        OXB_EPI(V_REQUANT_LEAN)
        OXB_EPI(V_REQUANT_LEAN_DYN)
        OXB_EPI(20)
        OXB_EPI(21)
        OXB_EPI(22)
        OXB_EPI(23)
        OXB_EPI(24)
        default:
          if (split) epilogue_role<BN, 25, true>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);
          else epilogue_role<BN, 25, false>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);
          break;
      }
    } else {
      switch (p.variant) {
        OXB_EPI(0)
        OXB_EPI(1)
        OXB_EPI(2)
        OXB_EPI(3)
        OXB_EPI(4)
        OXB_EPI(5)
        OXB_EPI(14)
        OXB_EPI(15)
        OXB_EPI(16)
        OXB_EPI(17)
        OXB_EPI(18)
        default:
          if (split) epilogue_role<BN, 19, true>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);
          else epilogue_role<BN, 19, false>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles);
          break;
      }
    }
#undef OXB_EPI
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the CTA's shared memory goes away
    long long start = clock64();
    while (clock64() - start < 2000000LL) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
                                   const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_encode_once;

void load_encoders() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      g_encode_tiled = (EncodeTiledFn)fn;
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      g_encode_im2col = (EncodeIm2colFn)fn;
    (void)cudaGetLastError();
  });
}

int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) cached = n;
    else cached = 148;
  }
  return cached;
}

CUtensorMapSwizzle swizzle_enum(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

uint32_t make_idesc(int kind, bool a_signed, bool b_signed, int bn) {
  uint32_t d = 0;
  if (kind == 0) {
    d |= 2u << 4;                      // accumulator: s32
    d |= (a_signed ? 1u : 0u) << 7;    // A: 0 = u8, 1 = s8
    d |= (b_signed ? 1u : 0u) << 10;   // B
  } else {
    d |= 1u << 4;  // accumulator: f32
    d |= 2u << 7;  // A: tf32
    d |= 2u << 10; // B: tf32
  }
  // bits 15/16: A and B are K-major (0)
  d |= (uint32_t)(bn >> 3) << 17;
  d |= (uint32_t)(BLOCK_M >> 4) << 24;
  return d;
}

template <int BN, int KIND>
void launch_t(const KParams& kp, int grid, size_t smem, cudaStream_t s) {
  static bool attr_set = false;
  static size_t attr_smem = 0;
  if (!attr_set || smem > attr_smem) {
    OXB_CUDA(cudaFuncSetAttribute(umma_conv_kernel<BN, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set = true;
    attr_smem = smem;
  }
  // Programmatic dependent launch: this grid may be scheduled while its predecessor in the stream drains, so
  // that its prologue (barrier setup, TMEM allocation) overlaps the predecessor's tail; it touches no global
  // memory before griddepcontrol.wait, which returns only once the predecessor has completed and flushed.
  static const bool pdl = std::getenv("OXB200_NO_PDL") == nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  OXB_CUDA(cudaLaunchKernelEx(&cfg, umma_conv_kernel<BN, KIND>, kp));
}

}  // namespace

struct UmmaPlan {
  KParams kp;
  int bn;
  int kind;
  int grid;
  size_t smem;
  char desc[160];
  void* ws = nullptr;        // split-K workspace and arrival counters, owned by the plan
  void* ws_count = nullptr;
};

bool umma_available() {
  load_encoders();
  return g_encode_tiled != nullptr && g_encode_im2col != nullptr;
}

bool umma_overlapping_positions_ok() {
  static int state = -1;
  if (state >= 0) return state == 1;
  load_encoders();
  state = 0;
  if (!g_encode_im2col) return false;
  // the shape of the 8-bit stem: 64-lane windows 16 lanes apart; nothing is read through this map
  CUtensorMap tm;
  cuuint64_t gdim[4] = {64, 112, 112, 2};
  cuuint64_t gstr[3] = {16, 115 * 16, 112 * 115 * 16};
  int lower[2] = {0, -2}, upper[2] = {0, -2};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult rc = g_encode_im2col(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, reinterpret_cast<void*>(uintptr_t(1) << 30), gdim, gstr, lower, upper, 64, BLOCK_M,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  state = rc == CUDA_SUCCESS ? 1 : 0;
  return state == 1;
}

int umma_channel_block(int C, int kind) {
  int es = kind == 0 ? 1 : 4;
  int64_t row = (int64_t)C * es;
  if (row % 128 == 0) return 128 / es;
  if (row == 64) return 64 / es;
  if (row == 32) return 32 / es;
  return 0;
}

UmmaPlan* umma_plan_create(const void* x, DT x_dt, const void* w_packed, DT w_dt, void* out, const ConvShape& cs, const Epilogue& e, int kind,
                           std::string* why) {
  auto no = [&](const char* msg) -> UmmaPlan* {
    if (why) *why = msg;
    return nullptr;
  };
  load_encoders();
  if (!g_encode_tiled || !g_encode_im2col) return no("tensor-map encoders unavailable in this driver");
  if (cs.group != 1) return no("grouped convolution");
  if (kind == 0) {
    if (!(x_dt == DT::U8 || x_dt == DT::I8) || !(w_dt == DT::I8 || w_dt == DT::U8)) return no("operands are not 8-bit integers");
    if (e.mode == EPI_F32) return no("integer kind needs an integer epilogue");
  } else {
    if (x_dt != DT::F32 || w_dt != DT::F32 || e.mode != EPI_F32) return no("tf32 kind needs f32 operands and a float epilogue");
  }
  const int es = kind == 0 ? 1 : 4;
  const int cb = umma_channel_block(cs.C, kind);
  if (cb == 0) return no("channel count is not a multiple of a 32/64/128-byte block");
  const int swz = cb * es;
  const int64_t M = cs.M();
  if (M <= 0 || M > 0x7fffffffLL || cs.OC <= 0) return no("empty or oversized problem");
  if (((uintptr_t)x & 127) || ((uintptr_t)w_packed & 127) || ((uintptr_t)out & 15)) return no("operand base address is not aligned");
  const bool gemm_like = cs.R == 1 && cs.S == 1 && cs.sh == 1 && cs.sw == 1 && cs.pt == 0 && cs.pl == 0 && cs.pb == 0 && cs.pr == 0 &&
                         cs.x_pixel_stride == 0 && cs.x_row_pixels == 0;
  if (!gemm_like) {
    // im2col corners and offsets are 8-bit quantities for two spatial dimensions
    int up_w = cs.pr - (cs.S - 1) * cs.dw, up_h = cs.pb - (cs.R - 1) * cs.dh;
    if (cs.pl > 127 || cs.pt > 127 || up_w < -128 || up_h < -128 || up_w > 127 || up_h > 127) return no("padding outside the im2col corner range");
    if ((cs.S - 1) * cs.dw > 255 || (cs.R - 1) * cs.dh > 255) return no("filter extent outside the im2col offset range");
    if (cs.sw > 8 || cs.sh > 8) return no("stride above the TMA traversal-stride limit");
  }
  if (e.x_zp_rows || e.n_w_zp > 0) return no("per-row or weight zero points need the direct kernel");

  // Tile width.  Measured on B200 (1.965 GHz): a tcgen05.mma of 32 bytes of K takes N/2 cycles
  // of the tensor pipe but cannot be issued faster than one per ~56 cycles; one SM fills its
  // shared memory from L2 at about 95 GB/s when all SMs do so; the fused epilogue costs about
  // 0.08 ns per output for requantisation and 0.03 ns for the float variants, spread over eight
  // warps.  The three overlap (ring of stages, two accumulators), so a tile takes the longest of
  // them, the kernel runs ceil(tiles / SMs) rounds of tiles, and the last tile's epilogue is
  // not hidden.  Pick the width that minimises that estimate; ties go to the wider tile (fewer
  // re-reads of the activations).
  // Split K: when even the narrowest useful tiling leaves most SMs without a tile and K is long, `splits`
  // CTAs share a (wider) tile, each running a slice of K; the slices meet in an L2-resident workspace.  It is
  // only considered when every slice gets its own SM in one round and at least eight K blocks.
  const int sms = sm_count();
  const int64_t m_tiles = ceil_div(M, BLOCK_M);
  const int bn_max = cs.OC <= 32 ? 32 : (cs.OC <= 64 ? 64 : (cs.OC <= 128 ? 128 : 256));
  const int64_t k_iters_host = (int64_t)cs.R * cs.S * (cs.C / cb);
  int bn = bn_max, splits = 1;
  {
    const double k_bytes = (double)cs.K() * es;
    const double k_steps = k_bytes / 32.0;
    const double ns_out = e.mode == EPI_F32 ? 0.03e-9 : 0.08e-9;
    const char* env_split = std::getenv("OXB200_UMMA_SPLITK");  // upper bound on the slices; "1": never split (for comparisons)
    const int max_split = env_split ? std::max(1, std::atoi(env_split)) : 8;
    double best = 1e30;
    for (int cand = bn_max; cand >= 32; cand /= 2) {
      const double tiles = (double)m_tiles * (double)ceil_div(cs.OC, cand);
      for (int sp = 1; sp <= max_split; ++sp) {
        if (sp > 1 && (tiles * sp > sms || k_iters_host / sp < 8)) break;
        const double rounds = std::ceil(tiles * sp / sms);
        const double t_mma = k_steps * std::max(56.0, cand / 2.0) / 1.965e9 / sp;
        const double t_feed = (double)(BLOCK_M + cand) * k_bytes / 95e9 / sp;
        const double t_epi = (double)BLOCK_M * cand * ns_out;
        // measured: a split launch costs about 10 us more than an unsplit one before its first K block pays
        // back (the slices' accumulators go through the workspace, and the finishing epilogues are not overlapped)
        const double t_split = sp > 1 ? 10e-6 : 0.0;
        const double t = rounds * std::max(t_mma, std::max(t_feed, t_epi)) + t_epi + t_split;
        if (t < best * 0.97) {
          best = t;
          bn = cand;
          splits = sp;
        }
      }
    }
  }
  const int64_t n_tiles = ceil_div(cs.OC, bn);
  if (m_tiles * n_tiles > 0x7fffffffLL) return no("grid too large");

  UmmaPlan* pl = new UmmaPlan();
  std::memset(&pl->kp, 0, sizeof(KParams));
  KParams& kp = pl->kp;
  CUtensorMapDataType dtype = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult rc;
  if (gemm_like) {
    cuuint64_t gdim[2] = {(cuuint64_t)cs.C, (cuuint64_t)M};
    cuuint64_t gstr[1] = {(cuuint64_t)cs.C * es};
    cuuint32_t box[2] = {(cuuint32_t)cb, (cuuint32_t)BLOCK_M};
    cuuint32_t estr[2] = {1, 1};
    rc = g_encode_tiled(&kp.tmA, dtype, 2, const_cast<void*>(x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    kp.a_im2col = 0;
  } else {
    const int64_t pix = cs.x_pixel_stride > 0 ? cs.x_pixel_stride : cs.C, row = (cs.x_row_pixels > 0 ? cs.x_row_pixels : cs.W) * pix;
    cuuint64_t gdim[4] = {(cuuint64_t)cs.C, (cuuint64_t)cs.W, (cuuint64_t)cs.H, (cuuint64_t)cs.N};
    cuuint64_t gstr[3] = {(cuuint64_t)pix * es, (cuuint64_t)row * es, (cuuint64_t)cs.H * row * es};
    int lower[2] = {-cs.pl, -cs.pt};
    int upper[2] = {cs.pr - (cs.S - 1) * cs.dw, cs.pb - (cs.R - 1) * cs.dh};
    cuuint32_t estr[4] = {1, (cuuint32_t)cs.sw, (cuuint32_t)cs.sh, 1};
    rc = g_encode_im2col(&kp.tmA, dtype, 4, const_cast<void*>(x), gdim, gstr, lower, upper, (cuuint32_t)cb, (cuuint32_t)BLOCK_M, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    kp.a_im2col = 1;
    // Drivers up to CUDA 13.1 mis-encode im2col maps of tensors smaller than 128 KiB; the
    // published workaround clears bit 21 of the second descriptor word.
    int drv = 0;
    if (rc == CUDA_SUCCESS && cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010) {
      size_t bytes = (size_t)cs.N * cs.H * row * es;
      if (bytes < 131072) reinterpret_cast<uint64_t*>(&kp.tmA)[1] &= ~(1ull << 21);
    }
  }
  if (rc != CUDA_SUCCESS) {
    delete pl;
    return no("activation tensor map rejected by the driver");
  }
  {
    const int64_t ktot = cs.K();
    cuuint64_t gdim[2] = {(cuuint64_t)ktot, (cuuint64_t)cs.OC};
    cuuint64_t gstr[1] = {(cuuint64_t)ktot * es};
    cuuint32_t box[2] = {(cuuint32_t)cb, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    rc = g_encode_tiled(&kp.tmB, dtype, 2, const_cast<void*>(w_packed), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      delete pl;
      return no("weight tensor map rejected by the driver");
    }
  }
  {
    // output tile store through TMA when rows are 16-byte granular
    const size_t oes = dt_size(e.out_dt);
    // at most one epilogue warp's share of a row; one run when K is split (any slice may finish any run)
    const size_t row_bytes = splits > 1 ? 32 * oes : std::min<size_t>(128, (size_t)std::max(bn / 64, 1) * 32 * oes);
    kp.out_tma = 0;
    kp.out_row_bytes = (int)row_bytes;
    if (((size_t)cs.OC * oes) % 16 == 0 && ((uintptr_t)out & 15) == 0 && row_bytes >= 32 && (row_bytes & (row_bytes - 1)) == 0) {
      CUtensorMapDataType odt = oes == 4 ? (e.out_dt == DT::F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_INT32)
                                         : (oes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
      cuuint64_t gdim[2] = {(cuuint64_t)cs.OC, (cuuint64_t)M};
      cuuint64_t gstr[1] = {(cuuint64_t)cs.OC * oes};
      cuuint32_t box[2] = {(cuuint32_t)(row_bytes / oes), 32};
      cuuint32_t estr[2] = {1, 1};
      CUresult ro = g_encode_tiled(&kp.tmO, odt, 2, out, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum((int)row_bytes),
                                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (ro == CUDA_SUCCESS) kp.out_tma = 1;
    }
  }
  {
    const char* dbg = std::getenv("OXB200_UMMA_DEBUG");
    kp.dbg = dbg ? std::atoi(dbg) : 0;
    if (dbg && std::atoi(dbg) == 4) {
      kp.dbg = 0;
      kp.out_tma = 0;
    }
  }
  kp.M = (int)M;
  kp.OC = cs.OC;
  kp.P = cs.P;
  kp.Q = cs.Q;
  kp.S = cs.S;
  kp.sh = cs.sh;
  kp.sw = cs.sw;
  kp.pt = cs.pt;
  kp.pl = cs.pl;
  kp.dh = cs.dh;
  kp.dw = cs.dw;
  kp.taps = cs.R * cs.S;
  kp.cblocks = cs.C / cb;
  kp.cb_elems = cb;
  kp.swizzle_bytes = swz;
  kp.n_tiles = (int)n_tiles;
  kp.m_tiles = (int)m_tiles;
  kp.idesc = make_idesc(kind, x_dt == DT::I8, w_dt == DT::I8, bn);
  // K blocks per stage: up to four small ones share a barrier round trip, as long as a stage stays
  // within 64 KB (the ring then still has three stages)
  const size_t kb_bytes = (size_t)(BLOCK_M + bn) * swz;
  int kpb = 1;
  while (kpb < 4 && (size_t)(kpb * 2) * kb_bytes <= 64 * 1024 && kpb * 2 <= k_iters_host) kpb *= 2;
  if (const char* env = std::getenv("OXB200_UMMA_KPB")) kpb = std::max(1, std::min(4, std::atoi(env)));
  kp.kpb = kpb;
  // slices of K: whole stages each, none empty
  kp.splits = 1;
  kp.k_per = (int)k_iters_host;
  if (splits > 1) {
    const int64_t k_per = ceil_div(ceil_div(k_iters_host, (int64_t)splits), (int64_t)kpb) * kpb;
    const int64_t eff = ceil_div(k_iters_host, k_per);
    if (eff > 1) {
      const size_t ws_words = (size_t)m_tiles * n_tiles * eff * BLOCK_M * bn;
      const size_t cnt = (size_t)m_tiles * n_tiles * EPI_WARPS * 4;
      if (cudaMalloc(&pl->ws, ws_words * 4) == cudaSuccess && cudaMalloc(&pl->ws_count, cnt * sizeof(unsigned int)) == cudaSuccess &&
          cudaMemset(pl->ws_count, 0, cnt * sizeof(unsigned int)) == cudaSuccess) {
        kp.splits = (int)eff;
        kp.k_per = (int)k_per;
        kp.ws = (uint32_t*)pl->ws;
        kp.ws_count = (unsigned int*)pl->ws_count;
      } else {
        (void)cudaGetLastError();  // no workspace: run unsplit
      }
    }
  }
  const size_t stage_bytes = kb_bytes * kpb;
  // one persistent CTA per SM: the ring may use most of the 227 KB and runs on across tiles
  const size_t budget = 192 * 1024;
  int stages = (int)(budget / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) stages = 2;
  kp.stages = stages;
  kp.mode = e.mode;
  if (e.mode == EPI_F32) kp.variant = e.act * 2 + (e.round_tf32 ? 1 : 0) + (e.residual ? V_F32_RES : 0);
  else if (e.mode == EPI_REQUANT) {
    const bool no_fma = std::getenv("OXB200_REQUANT_F64") != nullptr;  // keeps the two-pass variant reachable for tests
    const bool fma = e.combined_fma_ok && !no_fma;
    const bool lean = fma && e.acc_abs_bound > 0 && e.acc_abs_bound < 16777216;
    if (e.x_zp_dev) kp.variant = lean ? V_REQUANT_LEAN_DYN : (fma ? V_REQUANT_FMA_DYN : V_REQUANT_DYN);
    else kp.variant = lean ? V_REQUANT_LEAN : (fma ? V_REQUANT_FMA : V_REQUANT);
  }
  else if (e.mode == EPI_DEQUANT) kp.variant = V_DEQUANT + (e.x_zp_dev ? 1 : 0) + 2 * e.dq_act;
  else kp.variant = e.x_zp_dev ? V_INT32_DYN : V_INT32;
  if (e.mode == EPI_F32 ? e.bias_f == nullptr : e.bias_i == nullptr) {
    if (pl->ws) cudaFree(pl->ws);
    if (pl->ws_count) cudaFree(pl->ws_count);
    delete pl;
    return no("the tensor-core epilogue needs a (padded) bias vector");
  }
  kp.bias_f = e.bias_f;
  kp.residual = e.residual;
  kp.dq_w_scale = e.dq_w_scale;
  kp.dq_x_scale = e.dq_x_scale_dev;
  kp.dq_bias = e.dq_bias;
  kp.act = e.act;
  kp.clip_lo = e.clip_lo;
  kp.clip_hi = e.clip_hi;
  kp.round_tf32 = e.round_tf32;
  kp.bias_i = e.bias_i;
  kp.wsum = e.x_zp_dev ? e.wsum : nullptr;
  kp.x_zp_dev = e.x_zp_dev;
  kp.combined = e.combined;
  kp.y_zp = e.y_zp;
  kp.lo = (e.relu_fused && e.lo < 0) ? 0 : e.lo;
  kp.hi = e.hi;
  kp.out_dt = (int)e.out_dt;
  kp.out = out;
  kp.err_flag = nullptr;
  pl->bn = bn;
  pl->kind = kind;
  pl->grid = (int)std::min<int64_t>(m_tiles * n_tiles * kp.splits, sms);
  pl->smem = (size_t)stages * stage_bytes + 1024;
  char split_note[24] = "";
  if (kp.splits > 1) snprintf(split_note, sizeof split_note, " splitK=%d", kp.splits);
  snprintf(pl->desc, sizeof pl->desc, "umma_%s M=%lld N=%d K=%lld tile=128x%dx%dB stages=%dx%d %s%s", kind == 0 ? "i8" : "tf32", (long long)M, cs.OC,
           (long long)cs.K(), bn, swz, stages, kpb, gemm_like ? "tiled" : "im2col", split_note);
  return pl;
}

// Batched f32 (TF32) products whose operands are strided windows of larger row-major matrices: item
// (outer, inner) multiplies A rows [outer*a_rb + inner*a_rh, +M) x columns [inner*a_ch, +K) by B rows
// [outer*b_rb + inner*b_rh, +N) x columns [inner*b_ch, +K) (B is [N][K], K contiguous) into out rows
// [outer*o_rb + inner*o_rh, +M) x columns [inner*o_ch, +N).  This is how attention reads Q, K and V straight
// out of the [tokens, hidden] outputs of their linears and writes the context back in that layout.
UmmaPlan* umma_plan_create_batched(const BatchedGemm& g, std::string* why) {
  auto no = [&](const char* msg) -> UmmaPlan* {
    if (why) *why = msg;
    return nullptr;
  };
  load_encoders();
  if (!g_encode_tiled) return no("tensor-map encoders unavailable in this driver");
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.outer <= 0 || g.inner <= 0) return no("empty problem");
  if (g.M % BLOCK_M != 0) return no("rows per item are not a multiple of 128");
  const int cb = umma_channel_block(g.K, 1);
  if (cb == 0) return no("K is not a multiple of a 32-byte block");
  if (g.N % 32 != 0) return no("columns per item are not a multiple of 32");
  int bn = 256;
  while (bn > 32 && g.N % bn != 0) bn /= 2;
  if (g.N % bn != 0) return no("columns per item do not tile");
  if ((g.a_ch % 4) || (g.b_ch % 4) || (g.o_ch % 4) || (g.a_cols % 4) || (g.b_cols % 4) || (g.o_cols % 4)) return no("column offsets are not 16-byte granular");
  if (((uintptr_t)g.a & 127) || ((uintptr_t)g.b & 127) || ((uintptr_t)g.out & 15)) return no("operand base address is not aligned");
  const int swz = cb * 4;
  const int64_t items = (int64_t)g.outer * g.inner, m_tiles = g.M / BLOCK_M, n_tiles = g.N / bn;
  if (items * m_tiles * n_tiles > 0x7fffffffLL) return no("grid too large");
  UmmaPlan* pl = new UmmaPlan();
  std::memset(&pl->kp, 0, sizeof(KParams));
  KParams& kp = pl->kp;
  const CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint32_t estr[2] = {1, 1};
  {
    cuuint64_t gdim[2] = {(cuuint64_t)g.a_cols, (cuuint64_t)g.a_rows};
    cuuint64_t gstr[1] = {(cuuint64_t)g.a_cols * 4};
    cuuint32_t box[2] = {(cuuint32_t)cb, (cuuint32_t)BLOCK_M};
    if (g_encode_tiled(&kp.tmA, dtype, 2, const_cast<void*>(g.a), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz),
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      delete pl;
      return no("A tensor map rejected by the driver");
    }
  }
  {
    cuuint64_t gdim[2] = {(cuuint64_t)g.b_cols, (cuuint64_t)g.b_rows};
    cuuint64_t gstr[1] = {(cuuint64_t)g.b_cols * 4};
    cuuint32_t box[2] = {(cuuint32_t)cb, (cuuint32_t)bn};
    if (g_encode_tiled(&kp.tmB, dtype, 2, const_cast<void*>(g.b), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz),
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      delete pl;
      return no("B tensor map rejected by the driver");
    }
  }
  {
    const size_t row_bytes = std::min<size_t>(128, (size_t)std::max(bn / 64, 1) * 32 * 4);
    kp.out_row_bytes = (int)row_bytes;
    cuuint64_t gdim[2] = {(cuuint64_t)g.o_cols, (cuuint64_t)g.o_rows};
    cuuint64_t gstr[1] = {(cuuint64_t)g.o_cols * 4};
    cuuint32_t box[2] = {(cuuint32_t)(row_bytes / 4), 32};
    if (g_encode_tiled(&kp.tmO, dtype, 2, g.out, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum((int)row_bytes),
                       CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      delete pl;
      return no("output tensor map rejected by the driver");
    }
    kp.out_tma = 1;  // the only store path of the batched form
  }
  kp.M = g.M;
  kp.OC = g.N;
  kp.P = kp.Q = kp.S = 1;
  kp.sh = kp.sw = kp.dh = kp.dw = 1;
  kp.taps = 1;
  kp.cblocks = g.K / cb;
  kp.cb_elems = cb;
  kp.swizzle_bytes = swz;
  kp.n_tiles = (int)n_tiles;
  kp.m_tiles = (int)m_tiles;
  kp.batched = 1;
  kp.splits = 1;
  kp.items = (int)items;
  kp.items_inner = g.inner;
  kp.a_rb = g.a_rb, kp.a_rh = g.a_rh, kp.a_ch = g.a_ch;
  kp.b_rb = g.b_rb, kp.b_rh = g.b_rh, kp.b_ch = g.b_ch;
  kp.o_rb = g.o_rb, kp.o_rh = g.o_rh, kp.o_ch = g.o_ch;
  kp.idesc = make_idesc(1, false, false, bn);
  const size_t kb_bytes = (size_t)(BLOCK_M + bn) * swz;
  int kpb = 1;
  while (kpb < 4 && (size_t)(kpb * 2) * kb_bytes <= 64 * 1024 && kpb * 2 <= kp.cblocks) kpb *= 2;
  kp.kpb = kpb;
  const size_t stage_bytes = kb_bytes * kpb;
  int stages = (int)((192 * 1024) / stage_bytes);
  stages = std::max(2, std::min(stages, MAX_STAGES));
  kp.stages = stages;
  kp.mode = EPI_F32;
  kp.variant = g.round_tf32 ? 1 : 0;
  kp.bias_f = g.zero_bias;
  kp.round_tf32 = g.round_tf32;
  kp.out_dt = (int)DT::F32;
  kp.out = g.out;
  pl->bn = bn;
  pl->kind = 1;
  pl->grid = (int)std::min<int64_t>(items * m_tiles * n_tiles, sm_count());
  pl->smem = (size_t)stages * stage_bytes + 1024;
  snprintf(pl->desc, sizeof pl->desc, "umma_tf32 batched %lldx(M=%d N=%d K=%d) tile=128x%dx%dB stages=%dx%d", (long long)items, g.M, g.N, g.K, bn, swz, stages, kpb);
  return pl;
}

void umma_plan_destroy(UmmaPlan* p) {
  if (!p) return;
  if (p->ws) cudaFree(p->ws);
  if (p->ws_count) cudaFree(p->ws_count);
  delete p;
}
void umma_plan_reset_after_error(UmmaPlan* p) {
  if (!p || !p->ws_count) return;
  const size_t cnt = (size_t)p->kp.m_tiles * p->kp.n_tiles * EPI_WARPS * 4;
  (void)cudaMemset(p->ws_count, 0, cnt * sizeof(unsigned int));
}
const char* umma_plan_desc(const UmmaPlan* p) { return p->desc; }

void umma_launch(const UmmaPlan* p, int* err_flag, cudaStream_t s) {
  KParams kp = p->kp;
  kp.err_flag = err_flag;
#ifdef OXB_UMMA_TRACE
  static long long* trace_dev = nullptr;
  if (!trace_dev) OXB_CUDA(cudaMalloc(&trace_dev, 64 * 16 * sizeof(long long)));
  OXB_CUDA(cudaMemsetAsync(trace_dev, 0, 64 * 16 * sizeof(long long), s));
  kp.trace = trace_dev;
#endif
#define OXB_UMMA_CASE(BN)                                             \
  case BN:                                                            \
    if (p->kind == 0) launch_t<BN, 0>(kp, p->grid, p->smem, s);       \
    else launch_t<BN, 1>(kp, p->grid, p->smem, s);                    \
    break;
  switch (p->bn) {
    OXB_UMMA_CASE(32)
    OXB_UMMA_CASE(64)
    OXB_UMMA_CASE(128)
    OXB_UMMA_CASE(256)
    default: OXB_FAIL("umma_launch: unsupported tile width %d", p->bn);
  }
#undef OXB_UMMA_CASE
  OXB_CUDA(cudaGetLastError());
#ifdef OXB_UMMA_TRACE
  if (std::getenv("OXB200_UMMA_TRACE")) {
    static long long host[64 * 16];
    OXB_CUDA(cudaStreamSynchronize(s));
    OXB_CUDA(cudaMemcpy(host, trace_dev, sizeof host, cudaMemcpyDeviceToHost));
    long long t0 = host[0];
    fprintf(stderr, "trace %s\n tile:  prod0 prod1 | mma0 accfree full0 issued | epi0 accfull done0 done3\n", p->desc);
    for (int t = 0; t < 40; ++t) {
      if (!host[t * 16 + 0] && !host[t * 16 + 2]) break;
      fprintf(stderr, " %3d:", t);
      for (int k = 0; k < 10; ++k) fprintf(stderr, " %7lld%s", host[t * 16 + k] ? host[t * 16 + k] - t0 : -1, (k == 1 || k == 5) ? " |" : "");
      if (t == 0 && host[10]) fprintf(stderr, "  last slice of tile 0: loads of run 0 %lld, its epilogue %lld, all runs %lld cycles", host[11] - host[10], host[12] - host[11], host[13] - host[10]);
      fprintf(stderr, "\n");
    }
    fprintf(stderr, " tile 3 per K block: prod_wait0 prod_wait1 prod_issued | mma_wait0 mma_wait1 mma_issued\n");
    for (int t = 40; t < 64; ++t) {
      if (!host[t * 16 + 0] && !host[t * 16 + 3]) break;
      fprintf(stderr, " %3d:", t - 40);
      for (int k = 0; k < 6; ++k) fprintf(stderr, " %7lld%s", host[t * 16 + k] ? host[t * 16 + k] - t0 : -1, k == 2 ? " |" : "");
      fprintf(stderr, "\n");
    }
  }
#endif
}

}  // namespace k
}  // namespace oxb
