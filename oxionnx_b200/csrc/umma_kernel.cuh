// tcgen05 implicit-GEMM convolution / GEMM for sm_100a: the device code and the launch templates.
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
//  * B tiles (output channels x the same K slice) are 2-D tiled TMA loads.
//  * No load uses cluster multicast: every CTA fetches its own tiles.
//  * One elected thread issues tcgen05.mma (kind::i8 with s32 accumulation, kind::tf32 or
//    kind::f16 with f32 accumulation) from shared-memory descriptors into TMEM accumulators
//    of BN columns; a ring stage carries up to four K blocks when they are small, so that the
//    barrier round trip and the fixed cost of each asynchronous instruction are paid per stage.
//  * CTA pairs (PAIR): two CTAs of a cluster share one 256 x 256 tile.  Each stages its own 128
//    rows of A and its own 128 rows of B (half of what a lone CTA stages per output), the even
//    CTA issues tcgen05.mma.cta_group::2 for both, and each drains the 128 x 256 accumulator
//    that lands in its own TMEM.  The pair's loads signal the even CTA's barrier; its commits
//    free the ring stage and publish the accumulator in both CTAs.
//  * Epilogue warps (sixteen for the integer kind, eight for the float kinds) read the
//    accumulator with tcgen05.ld (one output pixel per thread, 32 channels per load), apply the
//    fused epilogue in registers and hand the tile to TMA stores through swizzled staging rows.
//    A warp may only read the TMEM lanes 32 * (warp % 4) .. + 31, so the warps of a lane
//    quarter split a tile's channel runs, at least two runs per warp; when that leaves warps
//    over (tiles narrower than 256 channels) the warps form groups, each group drains a tile of
//    its own, and there are two accumulators per group (up to eight).
//  * Epilogue variants, one tile loop instantiated per variant: float bias / ReLU / clip /
//    SiLU / PRelu / TF32 rounding, optionally with a fused residual; exact ONNX requantisation
//    in one fused multiply-add per output (and an f64 two-pass form for scales outside its
//    proven range); int32 saturation; the dequantising chain of a dynamically quantised linear.
//  * Batched products (attention) address each item's operands and output as windows of larger
//    row-major matrices, so heads are read and written in place.
//  * The grid is launched with programmatic stream serialization and waits for its predecessor
//    (griddepcontrol.wait) only after its own prologue.
//  * Every mbarrier wait is bounded; on a timeout the kernel records an error code, lets its
//    copies land, frees its TMEM and returns, so the context stays usable.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "kernels.hpp"

namespace oxb {
namespace k {
namespace umma {

constexpr int BLOCK_M = 128;
constexpr int MAX_STAGES = 12;
constexpr int MAX_ACC = 8;
constexpr long long WAIT_CYCLES = 2000000000LL;  // ~1 s at 2 GHz

// Kinds of the contraction: operand storage and tensor-core instruction.
enum { KIND_I8 = 0, KIND_TF32 = 1, KIND_F16 = 2, KIND_BF16 = 3 };  // f16 and bf16 run the same kernel (kind::f16); the instruction descriptor tells them apart
// Epilogue warps per kind.  A 576-thread block leaves 96 registers per thread (five warps on two of the four
// schedulers, whose register files hold 16384 registers each), enough for the integer epilogues; the float
// kinds keep eight warps and 168 registers.
__host__ __device__ constexpr int epi_warps(int kind) { return kind == KIND_I8 ? 16 : 8; }

struct alignas(64) KParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmO;
  int out_tma, out_row_bytes;
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
  uint32_t stage_off;  // byte offset of the epilogue staging rows inside the dynamic shared memory (after the ring)
  // > 0: the layer has one channel tile and its whole packed weight matrix (this many bytes) stays in shared memory
  // in front of the ring for the life of the CTA; ring stages then hold activation blocks only
  uint32_t b_resident_bytes;
  // epilogue
  int mode;
  int variant;  // which epilogue_math instantiation runs
  const float* bias_f;
  const float* residual;  // f32 [M, OC] added after the bias, or null
  const float* slope;     // PRelu: per-channel slope, padded like the bias
  int act;
  float clip_lo, clip_hi;
  int round_tf32;
  const int32_t* bias_i;
  const float* bias_if;  // the folded integer bias as f32 lanes (exact), for the variant that adds it after the conversion
  const int32_t* wsum;
  const float* x_zp_dev;
  const float* combined;
  const float* dq_w_scale;   // dequantising epilogue: per-channel weight scale,
  const float* dq_x_scale;   // the activation's scale (one device lane),
  const float* dq_bias;      // per-channel f32 bias
  int y_zp, lo, hi;
  int out_dt;
  void* out;
  // f32 outputs only, or null: two ordered keys (see float_order_key) into which the kernel merges the minimum and
  // the maximum of everything it writes, for a DynamicQuantizeLinear that reads the output next
  unsigned int* minmax_keys;
  int* err_flag;
};

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
// The same test with a suspend-time hint (nanoseconds): the warp may stay parked in hardware that long before the
// instruction gives up, so a long wait costs few issue slots.
__device__ __forceinline__ uint32_t mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok;
}
// Bounded wait: false when the barrier did not flip within WAIT_CYCLES or another role aborted.  A waiting role
// shares its scheduler's issue slots with the epilogue warps, so the loop is kept to the parked test and a
// counter; the abort flag and the clock are looked at once per 32 attempts (an attempt returns within a few
// microseconds at the latest, so an abort is seen within a fraction of a millisecond and the limit holds).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
#pragma unroll 1
    for (int attempt = 0; attempt < 32; ++attempt)
      if (mbar_try_wait_parked(bar, parity, 4000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > WAIT_CYCLES) return false;
  }
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// arrival on a barrier of any CTA of the cluster (address from mapa)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
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
// The same two loads issued by a CTA of a pair: the data lands in the issuing CTA's shared memory, the bytes are
// counted on `bar`, a shared::cluster address that names the even CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
               "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h, int n, uint16_t off_w,
                                                         uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(
          dst),
      "l"((uint64_t)map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Makes `bar` track the completion of every tcgen05.mma this thread has issued so far.
template <bool PAIR>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if (PAIR) asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  else asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// The MMAs of one K block (1, 2 or 4 instructions of 32 bytes of K each) in one asm block: the
// 64-bit descriptors are assembled from a 32-bit low word that advances by 2 (16-byte units) per
// instruction and a constant high word, so the issuing thread spends a handful of integer
// instructions per K block.
#define OXB_MMA_BLOCK(GROUP, KINDSTR)                                                                       \
  asm volatile(                                                                                             \
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"                                 \
      "setp.ne.b32 p, %5, 0;\n\tsetp.ne.b32 q, 1, 0;\n\t"                                                   \
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"                                                  \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %4, p;\n\t"                         \
      "setp.lt.u32 p, %6, 2;\n\t@p bra DONE_%=;\n\t"                                                        \
      "add.u32 la, %1, 2;\n\tadd.u32 lb, %2, 2;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                         \
      "setp.lt.u32 p, %6, 4;\n\t@p bra DONE_%=;\n\t"                                                        \
      "add.u32 la, %1, 4;\n\tadd.u32 lb, %2, 4;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                         \
      "add.u32 la, %1, 6;\n\tadd.u32 lb, %2, 6;\n\tmov.b64 da, {la, %3};\n\tmov.b64 db, {lb, %3};\n\t"     \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %4, q;\n\t"                         \
      "DONE_%=:\n\t}" ::"r"(tmem_d),                                                                        \
      "r"(lo_a), "r"(lo_b), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(mmas)                            \
      : "memory")

template <int KIND, bool PAIR>
__device__ __forceinline__ void tc_mma_block(uint32_t tmem_d, uint32_t lo_a, uint32_t lo_b, uint32_t desc_hi, uint32_t idesc, uint32_t accumulate,
                                             uint32_t mmas) {
  if (PAIR) {
    if (KIND == KIND_I8) OXB_MMA_BLOCK("2", "i8");
    else if (KIND == KIND_TF32) OXB_MMA_BLOCK("2", "tf32");
    else OXB_MMA_BLOCK("2", "f16");
  } else {
    if (KIND == KIND_I8) OXB_MMA_BLOCK("1", "i8");
    else if (KIND == KIND_TF32) OXB_MMA_BLOCK("1", "tf32");
    else OXB_MMA_BLOCK("1", "f16");
  }
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

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, naming the registers a pending read lands in: nothing that uses them may be scheduled above it.
// Neither this nor the read itself is a compiler barrier for memory: the per-channel parameter loads of the run's
// math may be started above the wait, so that their latency (the top stall of the short-K layers) overlaps it.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :);
}

// Monotone map from f32 to u32: integer atomicMin / atomicMax on the keys give the exact float extrema.
__device__ __forceinline__ uint32_t float_order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ---- fused epilogue math ------------------------------------------------------------------
// One variant per (mode, activation, rounding) combination, chosen once per kernel, so that
// the 32 per-channel computations inside are straight-line code with full instruction-level
// parallelism.  Per-channel parameters are read with 16-byte read-only loads; the host pads
// every parameter vector to a multiple of 256 channels, so no bounds checks are needed here.
//
// Float variants: V_F32_BASE + 2 * act + round_tf32, act 0 none, 1 relu, 2 clip, 3 silu, 4 prelu (0..9), the
// same with a fused residual from V_F32_RES (10..19).  Integer variants follow.
enum {
  V_F32_BASE = 0,
  V_F32_RES = 10,
  V_REQUANT = 20,
  V_REQUANT_DYN = 21,
  V_INT32 = 22,
  V_INT32_DYN = 23,
  V_REQUANT_FMA = 24,
  V_REQUANT_FMA_DYN = 25,
  V_REQUANT_LEAN = 26,
  V_REQUANT_LEAN_DYN = 27,
  V_REQUANT_FBIAS = 28,  // LEAN with the bias added as a float after the conversion
  V_REQUANT_PACKED = 29, // FBIAS with the saturation done on packed 16-bit lanes (8-bit outputs of bounded magnitude)
  V_DEQUANT = 30         // 30..35: dequantising variants, + (dynamic zero point ? 1 : 0) + 2 * activation
};

__device__ __forceinline__ float act_f32(int act, float f, float slope, float lo, float hi) {
  if (act == 1) return fmaxf(f, 0.f);
  if (act == 2) return fminf(fmaxf(f, lo), hi);
  if (act == 3) return __fdiv_rn(f, __fadd_rn(1.0f, expf(-f)));     // silu: x / (1 + exp(-x)) (nn/activations.rs:271)
  if (act == 4) return f >= 0.f ? f : __fmul_rn(f, slope);          // prelu (nn/activations.rs:100)
  return f;
}

// Packs 32 f32 results into the output type: f32 (32 words), f16 or bf16 (16 words).  The tf32 kind only writes
// f32: the choice is made at compile time there, so that the packed words of a run have one definition each (a
// run-time choice between the 32-word and the 16-word form costs a select per word in an issue-bound loop).
template <int KIND>
__device__ __forceinline__ void pack_float(const float (&f)[4], int j4, int out_dt, uint32_t (&w)[32]) {
  if (KIND == KIND_TF32) {
#pragma unroll
    for (int e = 0; e < 4; ++e) w[4 * j4 + e] = __float_as_uint(f[e]);
    return;
  }
  if (out_dt == (int)DT::F16) {
    __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
    w[2 * j4] = *reinterpret_cast<uint32_t*>(&a);
    w[2 * j4 + 1] = *reinterpret_cast<uint32_t*>(&b);
  } else if (out_dt == (int)DT::BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    w[2 * j4] = *reinterpret_cast<uint32_t*>(&a);
    w[2 * j4 + 1] = *reinterpret_cast<uint32_t*>(&b);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) w[4 * j4 + e] = __float_as_uint(f[e]);
  }
}

template <int KIND, int ACT, int RT, bool RES>
__device__ __forceinline__ void math_f32(const KParams& p, const uint32_t (&v)[32], const float* __restrict__ bias, const float* __restrict__ slope,
                                         const float* __restrict__ res, uint32_t (&w)[32]) {
  // this pixel's 32 channels of the residual: one full 128-byte line per thread, all eight loads in flight
  // together before the first is used
  float4 rv[RES ? 8 : 1];
  if (RES) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) rv[j4] = res != nullptr ? __ldg(reinterpret_cast<const float4*>(res) + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const float4 b = __ldg(reinterpret_cast<const float4*>(bias) + j4);
    const float bb[4] = {b.x, b.y, b.z, b.w};
    float rr[4] = {0.f, 0.f, 0.f, 0.f};
    if (RES) rr[0] = rv[j4].x, rr[1] = rv[j4].y, rr[2] = rv[j4].z, rr[3] = rv[j4].w;
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    if (ACT == 4) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(slope) + j4);
      ss[0] = s.x, ss[1] = s.y, ss[2] = s.z, ss[3] = s.w;
    }
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      f[e] = __uint_as_float(v[4 * j4 + e]) + bb[e];
      if (RES) f[e] = __fadd_rn(f[e], rr[e]);
      f[e] = act_f32(ACT, f[e], ss[e], p.clip_lo, p.clip_hi);
      if (RT) f[e] = round_tf32(f[e]);
    }
    pack_float<KIND>(f, j4, p.out_dt, w);
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
// FBIAS (needs that bound too, which also covers the raw sum and the folded bias on their own): the raw
// accumulator is converted first and the bias, held as f32 lanes, is added as a float -- both terms and their
// sum are integers below 2^24, so the addition is exact; it runs on the FMA pipe instead of the integer pipe,
// which is the busier one in this epilogue.
template <bool DYN, bool FALLBACK, bool FBIAS>
__device__ __forceinline__ void math_requant_fma(const KParams& p, const uint32_t (&v)[32], const int32_t* __restrict__ bias,
                                                 const float* __restrict__ bias_f, const int32_t* __restrict__ wsum, const float* __restrict__ comb, int xz,
                                                 size_t esz, uint32_t (&w)[32]) {
  const float magic = 12582912.0f;  // 1.5 * 2^23
  const float magic_zp = magic + (float)p.y_zp, flo = magic + (float)p.lo, fhi = magic + (float)p.hi;
  // eight channels at a time, packed at once: few values are live together
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float amax = 0.f;
    uint32_t sb[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j4 = 2 * g + h;
      float a[4];
      if (FBIAS) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(bias_f) + j4);
        a[0] = __fadd_rn(__int2float_rn((int32_t)v[4 * j4]), b.x);
        a[1] = __fadd_rn(__int2float_rn((int32_t)v[4 * j4 + 1]), b.y);
        a[2] = __fadd_rn(__int2float_rn((int32_t)v[4 * j4 + 2]), b.z);
        a[3] = __fadd_rn(__int2float_rn((int32_t)v[4 * j4 + 3]), b.w);
      } else {
        const int4 b = __ldg(reinterpret_cast<const int4*>(bias) + j4);
        const int bb[4] = {b.x, b.y, b.z, b.w};
        int ss[4] = {0, 0, 0, 0};
        if (DYN) {
          const int4 sv = __ldg(reinterpret_cast<const int4*>(wsum) + j4);
          ss[0] = sv.x, ss[1] = sv.y, ss[2] = sv.z, ss[3] = sv.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int32_t acc = (int32_t)v[4 * j4 + e] + bb[e];
          if (DYN) acc -= xz * ss[e];
          a[e] = __int2float_rn(acc);
        }
      }
      const float4 c = __ldg(reinterpret_cast<const float4*>(comb) + j4);
      const float cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (FALLBACK) amax = fmaxf(amax, fabsf(a[e]));
        sb[4 * h + e] = __float_as_uint(fminf(fmaxf(fmaf(a[e], cc[e], magic_zp), flo), fhi));
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

// Two f32 operations in one instruction (add.rn.f32x2 / fma.rn.f32x2): the same IEEE results lane by lane, half
// the issue slots.
__device__ __forceinline__ void add2(float& x0, float& x1, float y0, float y1) {
  uint64_t a, b, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(x0), "f"(x1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(y0), "f"(y1));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(d));
}
__device__ __forceinline__ void fma2(float& x0, float& x1, float y0, float y1, float z) {
  uint64_t a, b, c, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(x0), "f"(x1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(y0), "f"(y1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c) : "f"(z));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(d));
}

// The one-FMA requantisation (see math_requant_fma; the float-bias form) for 8-bit outputs whose magnitude the
// host has bounded below 2^15 from the weights and the scales: the rounded result sits in the low mantissa bits
// of s = fma(a, c, 1.5 * 2^23 + zp), and because 1.5 * 2^23 has sixteen zero low bits, the low half-word of s is
// the result itself as a two's-complement int16.  Two results are packed into one register and saturated together
// with one packed min/max (a single instruction when the lower bound is 0, as behind a fused Relu), then four
// are packed into a word: 2.25 integer-pipe instructions per output instead of 3.75.  Bit-identical to the
// unpacked form wherever that bound holds, which is checked per layer at plan time.
template <bool RELU>
__device__ __forceinline__ void math_requant_packed(const KParams& p, const uint32_t (&v)[32], const float* __restrict__ bias_f,
                                                    const float* __restrict__ comb, uint32_t (&w)[32]) {
  const float magic_zp = 12582912.0f + (float)p.y_zp;
  const uint32_t lo2 = ((uint32_t)p.lo & 0xffffu) * 0x00010001u, hi2 = ((uint32_t)p.hi & 0xffffu) * 0x00010001u;
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const float4 b = __ldg(reinterpret_cast<const float4*>(bias_f) + j4);
    const float4 c = __ldg(reinterpret_cast<const float4*>(comb) + j4);
    float a0 = __int2float_rn((int32_t)v[4 * j4]), a1 = __int2float_rn((int32_t)v[4 * j4 + 1]);
    float a2 = __int2float_rn((int32_t)v[4 * j4 + 2]), a3 = __int2float_rn((int32_t)v[4 * j4 + 3]);
    add2(a0, a1, b.x, b.y);
    add2(a2, a3, b.z, b.w);
    fma2(a0, a1, c.x, c.y, magic_zp);
    fma2(a2, a3, c.z, c.w, magic_zp);
    uint32_t p01 = __byte_perm(__float_as_uint(a0), __float_as_uint(a1), 0x5410);
    uint32_t p23 = __byte_perm(__float_as_uint(a2), __float_as_uint(a3), 0x5410);
    if (RELU) {
      p01 = __vimin_s16x2_relu(p01, hi2);
      p23 = __vimin_s16x2_relu(p23, hi2);
    } else {
      p01 = __vmins2(__vmaxs2(p01, lo2), hi2);
      p23 = __vmins2(__vmaxs2(p23, lo2), hi2);
    }
    w[j4] = __byte_perm(p01, p23, 0x6420);
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
template <int KIND, int VARIANT>
__device__ __forceinline__ void epilogue_chunk(const KParams& p, const uint32_t (&v)[32], int xz, int oc, size_t esz, const float* res, uint32_t (&w)[32]) {
  if constexpr (VARIANT < V_F32_RES) math_f32<KIND, VARIANT / 2, VARIANT & 1, false>(p, v, p.bias_f + oc, p.slope + oc, nullptr, w);
  else if constexpr (VARIANT < V_REQUANT) math_f32<KIND, (VARIANT - V_F32_RES) / 2, (VARIANT - V_F32_RES) & 1, true>(p, v, p.bias_f + oc, p.slope + oc, res, w);
  else if constexpr (VARIANT >= V_DEQUANT) {
    const float xs = __ldg(p.dq_x_scale);
    math_dequant<((VARIANT - V_DEQUANT) & 1) != 0, (VARIANT - V_DEQUANT) / 2>(p, v, p.bias_i + oc, p.wsum + oc, p.dq_w_scale + oc, p.dq_bias + oc, xz, xs, w);
  } else if constexpr (VARIANT == V_REQUANT) math_int<true, false>(p, v, p.bias_i + oc, nullptr, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_DYN) math_int<true, true>(p, v, p.bias_i + oc, p.wsum + oc, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_INT32) math_int<false, false>(p, v, p.bias_i + oc, nullptr, nullptr, xz, esz, w);
  else if constexpr (VARIANT == V_INT32_DYN) math_int<false, true>(p, v, p.bias_i + oc, p.wsum + oc, nullptr, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_FMA) math_requant_fma<false, true, false>(p, v, p.bias_i + oc, nullptr, nullptr, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_FMA_DYN) math_requant_fma<true, true, false>(p, v, p.bias_i + oc, nullptr, p.wsum + oc, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_LEAN) math_requant_fma<false, false, false>(p, v, p.bias_i + oc, nullptr, nullptr, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_LEAN_DYN) math_requant_fma<true, false, false>(p, v, p.bias_i + oc, nullptr, p.wsum + oc, p.combined + oc, xz, esz, w);
  else if constexpr (VARIANT == V_REQUANT_FBIAS) math_requant_fma<false, false, true>(p, v, nullptr, p.bias_if + oc, nullptr, p.combined + oc, xz, esz, w);
  else {
    if (p.lo == 0) math_requant_packed<true>(p, v, p.bias_if + oc, p.combined + oc, w);
    else math_requant_packed<false>(p, v, p.bias_if + oc, p.combined + oc, w);
  }
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
// `row_addr` is the lane's staging row, `xor_bits` its swizzle term (((row * pitch) >> 7) & (pitch / 16 - 1)): both
// are fixed for the life of the warp and computed once by the caller.
__device__ __forceinline__ void store_staged(const uint32_t (&w)[32], uint32_t row_addr, uint32_t xor_bits, int byte_off, int bytes) {
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

// Tile coordinates of a CTA's walk over the tile list (channel tile fastest) without a division per tile: the
// step splits once into whole rows of channel tiles and a remainder.  Used for the plain case (one item, no split
// reduction); the batched and split forms decode the tile number as before.
struct TileWalk {
  int m, n, dm, dn, n_tiles;
  __device__ __forceinline__ TileWalk(int tile0, int step, int n_tiles_) : n_tiles(n_tiles_) {
    m = tile0 / n_tiles_;
    n = tile0 - m * n_tiles_;
    dm = step / n_tiles_;
    dn = step - dm * n_tiles_;
  }
  __device__ __forceinline__ void next() {
    m += dm;
    n += dn;
    if (n >= n_tiles) {
      n -= n_tiles;
      ++m;
    }
  }
};

// How the epilogue warps of a block share tiles (see the file header).
template <int BN, int EW>
struct EpiShape {
  static constexpr int RUNS = BN / 32;                          // 32-channel runs of a tile
  static constexpr int WPQ_ALL = EW / 4;                        // warps per TMEM lane quarter
  // ... that share one tile: every warp takes at least two runs of a tile that has them, so that the per-tile
  // handshakes are paid once per two runs and a warp's staged rows (and its TMA store) are 64 bytes or more
  static constexpr int HALF_RUNS = RUNS >= 2 ? RUNS / 2 : 1;
  static constexpr int WPQ = WPQ_ALL < HALF_RUNS ? WPQ_ALL : HALF_RUNS;
  static constexpr int NG = WPQ_ALL / WPQ;                      // groups; tile number i of a CTA goes to group i % NG
  static constexpr int CPW = RUNS / WPQ;                        // runs per warp and tile
  static constexpr int NACC = 2 * NG;                           // accumulators: two per group
  static constexpr uint32_t TMEM_COLS = (NACC * BN) < 32 ? 32 : (NACC * BN);
  static_assert(NACC <= MAX_ACC && NACC * BN <= 512, "accumulators exceed the tensor memory of an SM");
};

// ---- epilogue role ------------------------------------------------------------------------
// Per run: TMEM read of the following run in flight, fused math, then either a swizzled copy into
// this warp's staging rows followed by one TMA store per `pitch` bytes of row, or direct 16-byte
// stores.  The accumulator is handed back to the MMA issuer as soon as this warp's last TMEM read
// has landed, before the last run's math.  `acc_empty` is the barrier address to arrive on: the
// CTA's own, or the even CTA's for a pair (a shared::cluster address).
template <int BN, int KIND, int VARIANT, bool SPLIT, bool PAIR>
__device__ __forceinline__ void epilogue_role(const KParams& p, int warp, int lane, uint32_t tmem_base, uint64_t* bar_acc_full,
                                              uint64_t* bar_acc_empty, uint32_t stage_addr, volatile int* abortp, int total_tiles, int tile0, int tile_step,
                                              int pair_rank) {
  constexpr int EW = epi_warps(KIND);
  using ES = EpiShape<BN, EW>;
  constexpr int CPW = ES::CPW;
  const int quarter = warp & 3;
  const int ew = warp - 2;
  const int slot = ew >> 2;               // 0 .. EW/4 - 1 within the lane quarter
  const int group = slot / ES::WPQ;       // which tiles this warp drains
  const int first = (slot % ES::WPQ) * CPW;
  int xz = 0;
  if (p.x_zp_dev) xz = __float2int_rn(*p.x_zp_dev);
  const size_t esz = (p.out_dt == (int)DT::F32 || p.out_dt == (int)DT::I32) ? 4 : ((p.out_dt == (int)DT::I16 || p.out_dt == (int)DT::F16 || p.out_dt == (int)DT::BF16) ? 2 : 1);
  const int chunk_bytes = 32 * (int)esz;
  const int pitch = p.out_row_bytes;  // staged row length: 32, 64 or 128 bytes, at most one warp's share of a row
  const int cpg = p.out_tma ? pitch / chunk_bytes : 1;  // runs per staged store: 1, 2 or 4
  const uint32_t stage_row_addr = stage_addr + (uint32_t)(lane * pitch);
  const uint32_t stage_xor = ((uint32_t)(lane * pitch) >> 7) & (uint32_t)(pitch / 16 - 1);
  uint32_t local = 0;
  const bool plain = !p.batched && p.splits == 1;
  // extrema of the f32 lanes this thread writes, when a DynamicQuantizeLinear reads the output next
  const bool track = p.minmax_keys != nullptr && esz == 4 && (VARIANT < V_REQUANT || VARIANT >= V_DEQUANT);
  float seen_min = INFINITY, seen_max = -INFINITY;
  TileWalk walk(tile0, tile_step, p.n_tiles);
  for (int t = tile0; t < total_tiles; t += tile_step, ++local, walk.next()) {
    if (ES::NG > 1 && (int)(local % ES::NG) != group) continue;
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
    const int tile_n = plain ? walk.n : tt % p.n_tiles, tile_m = plain ? walk.m : tt / p.n_tiles;
    const int m0 = tile_m * (PAIR ? 2 * BLOCK_M : BLOCK_M) + (PAIR ? pair_rank * BLOCK_M : 0), oc0 = tile_n * BN;
    const uint32_t buf = local % (uint32_t)ES::NACC;
    bool ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (local / (uint32_t)ES::NACC) & 1u, abortp);
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
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa(smem_u32(&bar_acc_empty[buf]), 0));
        else mbar_arrive(smem_u32(&bar_acc_empty[buf]));
      }
    };
    auto math = [&](const uint32_t(&v)[32], int ch) {
      const float* res = (VARIANT >= V_F32_RES && VARIANT < V_REQUANT && row_ok) ? p.residual + (size_t)m * p.OC + oc0 + ch * 32 : nullptr;
      epilogue_chunk<KIND, VARIANT>(p, v, xz, oc0 + ch * 32, esz, res, w);
      if (track && row_ok) {
        const int valid = p.OC - (oc0 + ch * 32);  // lanes of a ragged last run hold no output
        if (valid >= 32) {
          // two independent chains per bound, so that the 64 comparisons are not one dependent sequence
          float lo2 = __uint_as_float(w[0]), hi2 = lo2;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            seen_min = fminf(seen_min, __uint_as_float(w[j]));
            seen_max = fmaxf(seen_max, __uint_as_float(w[j]));
            lo2 = fminf(lo2, __uint_as_float(w[j + 1]));
            hi2 = fmaxf(hi2, __uint_as_float(w[j + 1]));
          }
          seen_min = fminf(seen_min, lo2);
          seen_max = fmaxf(seen_max, hi2);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) {
              seen_min = fminf(seen_min, __uint_as_float(w[j]));
              seen_max = fmaxf(seen_max, __uint_as_float(w[j]));
            }
        }
      }
    };
    auto store = [&](int ch) {
      if (p.out_tma) {
        const int in_group = (ch - first) & (cpg - 1);
        if (in_group == 0) {
          // the staging rows are rewritten: their previous store must have read them
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        }
        store_staged(w, stage_row_addr, stage_xor, in_group * chunk_bytes, chunk_bytes);
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

    if (first >= end) {  // no run of this tile is ours (a ragged last channel tile)
      release();
      continue;
    }
    if constexpr (SPLIT) {
      // Runs are taken in an order rotated by the slice index and each run has its own arrival counter, so the
      // slices of a tile finish different runs last and share the summing and the fused epilogue between them.
      constexpr bool kFloatAcc = VARIANT < V_REQUANT;
      const int split = t - tt * p.splits;
      // workspace of one slice: [lane quarter][run][16-byte piece j][lane], so that every store and load of a
      // warp covers 512 contiguous bytes (only warps with the same index in the other slices read it back)
      const uint4* tile_ws = reinterpret_cast<const uint4*>(p.ws + (size_t)tt * p.splits * (BLOCK_M * BN)) + (size_t)quarter * (BN / 32) * 256 + lane;
      constexpr size_t kSlice = (size_t)BLOCK_M * BN / 4;  // 16-byte pieces per slice
      uint4* mine = const_cast<uint4*>(tile_ws) + (size_t)split * kSlice;
      unsigned int* counters = p.ws_count + ((size_t)tt * EW + ew) * 4;
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
    } else {
      // One copy of the run's code in the loop, each run reading its own accumulator columns first.  Starting the
      // next run's TMEM read under this run's store was measured and is slower (102.6 us against 96.7 us on a 1x1
      // 64 -> 256 layer at M = 802816): the other epilogue warps of the scheduler hide the read's latency, and the
      // conditional read costs register moves at the loop's join.
#pragma unroll 1
      for (int c = first; c < end; ++c) {
        tmem_ld32_nowait(taddr + (uint32_t)c * 32u, va);
        tmem_ld_wait_for(va);
        if (c + 1 == end) release();
        math(va, c);
        store(c);
      }
    }
  }
  if (p.out_tma && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (track) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      seen_min = fminf(seen_min, __shfl_xor_sync(0xffffffffu, seen_min, off));
      seen_max = fmaxf(seen_max, __shfl_xor_sync(0xffffffffu, seen_max, off));
    }
    if (lane == 0) {
      if (seen_min != INFINITY) atomicMin(p.minmax_keys, float_order_key(seen_min));
      if (seen_max != -INFINITY) atomicMax(p.minmax_keys + 1, float_order_key(seen_max));
    }
  }
}

// ---- the kernel ---------------------------------------------------------------------------
// Persistent: one CTA per SM (one pair per two SMs) walks the tile list (channel tile fastest, so
// CTAs that share an activation tile run together and meet in L2).  The shared-memory ring and the
// TMEM accumulators are both pipelined across tiles: while the epilogue warps drain one
// accumulator, the MMA issuer fills the next and the producer is already loading further ahead.
template <int BN, int KIND, bool PAIR>
__global__ void __launch_bounds__(64 + 32 * epi_warps(KIND), 1) umma_conv_kernel(const __grid_constant__ KParams p) {
  constexpr int EW = epi_warps(KIND);
  using ES = EpiShape<BN, EW>;
  static_assert(!PAIR || BN == 256, "a pair shares a 256 x 256 tile");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_acc_full[MAX_ACC];
  __shared__ __align__(8) uint64_t bar_acc_empty[MAX_ACC];
  __shared__ __align__(8) uint64_t bar_b_resident;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int swz = p.swizzle_bytes;
  // rows of B a CTA stages per K block: the whole channel tile, or its own half of the pair's
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  const uint32_t a_bytes = (uint32_t)BLOCK_M * swz, b_bytes = (uint32_t)B_ROWS * swz;
  const bool b_res = !PAIR && p.b_resident_bytes != 0;
  const uint32_t kb_bytes = b_res ? a_bytes : a_bytes + b_bytes;  // one K block of the ring: activations, then weights
  const uint32_t stage_bytes = kb_bytes * (uint32_t)p.kpb;        // one ring stage
  const uint32_t b_res_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // resident weights (when used), then the ring
  const uint32_t tiles_base = b_res_base + (b_res ? p.b_resident_bytes : 0u);
  const int k_iters = p.taps * p.cblocks;
  const int total_tiles = p.m_tiles * p.n_tiles * (p.batched ? p.items : p.splits);
  const int pair_rank = PAIR ? (int)cluster_ctarank() : 0;
  const bool leader = pair_rank == 0;
  // work items: one per CTA, or one per pair
  const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), 1);
    }
    mbar_init(smem_u32(&bar_b_resident), 1);
    for (int i = 0; i < ES::NACC; ++i) {
      mbar_init(smem_u32(&bar_acc_full[i]), 1);
      // one arrival per epilogue warp of the group that drains it (of both CTAs for a pair)
      mbar_init(smem_u32(&bar_acc_empty[i]), (PAIR ? 2 : 1) * 4 * ES::WPQ);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(ES::TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(ES::TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the other CTA's barriers exist before anything signals them
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
    // a pair's copies are counted on the even CTA's barrier, which alone announces the bytes of both
    const uint32_t tx_per_kb = PAIR ? 2u * kb_bytes : kb_bytes;
    if (b_res && tile0 < total_tiles && lane == 0) {
      // the whole weight matrix of the (only) channel tile, once: K block i at b_res_base + i * b_bytes
      mbar_expect_tx(smem_u32(&bar_b_resident), p.b_resident_bytes);
      for (int i = 0; i < k_iters; ++i) tma_load_2d(b_res_base + (uint32_t)i * b_bytes, &p.tmB, smem_u32(&bar_b_resident), i * p.cb_elems, 0);
    }
    __syncwarp();
    const bool plain = !p.batched && p.splits == 1;
    TileWalk walk(tile0, tile_step, p.n_tiles);
    for (int t = tile0; t < total_tiles && ok; t += tile_step, walk.next()) {
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
      const int tile_n = plain ? walk.n : tt % p.n_tiles, tile_m = plain ? walk.m : tt / p.n_tiles;
      const int m0 = tile_m * (PAIR ? 2 * BLOCK_M : BLOCK_M) + (PAIR ? pair_rank * BLOCK_M : 0);
      const int oc0 = tile_n * BN + (PAIR ? pair_rank * B_ROWS : 0);
      int q0 = 0, p0 = 0, n0 = 0;
      if (p.a_im2col) {
        q0 = m0 % p.Q;
        int rest = m0 / p.Q;
        p0 = rest % p.P;
        n0 = rest / p.P;
      }
      const int w_base = q0 * p.sw - p.pl, h_base = p0 * p.sh - p.pt;
      int cb = it_begin % p.cblocks, sx = (it_begin / p.cblocks) % p.S, r = (it_begin / p.cblocks) / p.S;
      // A barrier round trip, an expect_tx and each TMA instruction cost the issuing thread on the
      // order of a hundred cycles, whatever the box size: a stage carries several K blocks when
      // they are small, so that those costs are paid once per stage.
      for (int it = it_begin; it < it_end; it += p.kpb) {
        bool got = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*abortp) {
            *abortp = 1;
            atomicExch(p.err_flag, 1);
          }
          ok = false;
          break;
        }
        const int blocks = min(p.kpb, it_end - it);
        const uint32_t full_local = smem_u32(&bar_full[stage]);
        const uint32_t full = PAIR ? mapa(full_local, 0) : full_local;
        if (lane == 0 && leader) mbar_expect_tx(full_local, tx_per_kb * (uint32_t)blocks);
        uint32_t a_dst = tiles_base + stage * stage_bytes;
        for (int g = 0; g < blocks; ++g, a_dst += kb_bytes) {
          if (lane == 0) {  // one thread issues: every operand of the copies is warp-uniform
            const int c_off = cb * p.cb_elems;
            if (PAIR) {
              if (p.a_im2col) tma_load_im2col_4d_pair(a_dst, &p.tmA, full, c_off, w_base, h_base, n0, (uint16_t)(sx * p.dw), (uint16_t)(r * p.dh));
              else tma_load_2d_pair(a_dst, &p.tmA, full, a_col0 + c_off, a_row0 + m0);
              tma_load_2d_pair(a_dst + a_bytes, &p.tmB, full, b_col0 + (it + g) * p.cb_elems, b_row0 + oc0);
            } else {
              if (p.a_im2col) tma_load_im2col_4d(a_dst, &p.tmA, full, c_off, w_base, h_base, n0, (uint16_t)(sx * p.dw), (uint16_t)(r * p.dh));
              else tma_load_2d(a_dst, &p.tmA, full, a_col0 + c_off, a_row0 + m0);
              if (!b_res) tma_load_2d(a_dst + a_bytes, &p.tmB, full, b_col0 + (it + g) * p.cb_elems, b_row0 + oc0);
            }
          }
          if (++cb == p.cblocks) {
            cb = 0;
            if (++sx == p.S) {
              sx = 0;
              ++r;
            }
          }
        }
        __syncwarp();
        if (++stage == (uint32_t)p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    // Tail: every stage this CTA filled has been consumed and its release has arrived here, so no arrival is
    // still on its way to this CTA's shared memory when the CTA ends.
    for (int i = 0; i < p.stages && ok; ++i) {
      bool got = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp);
      if (!__all_sync(0xffffffffu, got)) break;  // another role has recorded the cause
      if (++stage == (uint32_t)p.stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the even CTA of a pair issues for both) ----------------
    if (leader) {
      const uint32_t mmas = (uint32_t)(swz / 32);
      const uint64_t desc_rest = make_smem_desc(0, swz);
      const uint32_t desc_hi = (uint32_t)(desc_rest >> 32), desc_lo = (uint32_t)desc_rest;
      const uint32_t idesc = p.idesc;
      const uint32_t ring16 = tiles_base >> 4, stage16 = stage_bytes >> 4, kb16 = kb_bytes >> 4, a16_bytes = a_bytes >> 4;
      uint32_t stage = 0, phase = 0, a16 = ring16;
      uint32_t local = 0;
      bool ok = true;
      const uint32_t bres16 = b_res_base >> 4, b16_bytes = b_bytes >> 4;
      if (b_res && tile0 < total_tiles) {  // the resident weights have landed
        const bool got = mbar_wait(smem_u32(&bar_b_resident), 0u, abortp);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*abortp) {
            *abortp = 1;
            atomicExch(p.err_flag, 5);
          }
          ok = false;
        }
        tc_fence_after();
      }
      for (int t = tile0; t < total_tiles && ok; t += tile_step, ++local) {
        const uint32_t buf = local % (uint32_t)ES::NACC;
        const uint32_t acc_phase = (local / (uint32_t)ES::NACC) & 1u;
        // the epilogue must have drained this accumulator (free on its first use)
        bool got = mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_phase ^ 1u, abortp);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && !*abortp) {
            *abortp = 1;
            atomicExch(p.err_flag, 4);
          }
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * (uint32_t)BN;
        int it_begin = 0, it_end = k_iters;
        if (!p.batched && p.splits > 1) {
          it_begin = (t % p.splits) * p.k_per;
          it_end = min(k_iters, it_begin + p.k_per);
        }
        for (int it = it_begin; it < it_end; it += p.kpb) {
          got = mbar_wait(smem_u32(&bar_full[stage]), phase, abortp);
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
            const int blocks = min(p.kpb, it_end - it);
            uint32_t b16 = a16;
            for (int g = 0; g < blocks; ++g, b16 += kb16) {
              const uint32_t w16 = b_res ? bres16 + (uint32_t)(it + g) * b16_bytes : b16 + a16_bytes;
              tc_mma_block<KIND, PAIR>(tmem_d, desc_lo | (b16 & 0x3fffu), desc_lo | (w16 & 0x3fffu), desc_hi, idesc, (it + g) > it_begin ? 1u : 0u, mmas);
            }
            // frees the stage, in both CTAs of a pair, once these MMAs have read it
            const uint32_t e = smem_u32(&bar_empty[stage]);
            if (PAIR) {
              tc_commit<true>(mapa(e, 0));
              tc_commit<true>(mapa(e, 1));
            } else {
              tc_commit<false>(e);
            }
          }
          __syncwarp();
          a16 += stage16;
          if (++stage == (uint32_t)p.stages) {
            stage = 0;
            phase ^= 1u;
            a16 = ring16;
          }
        }
        if (ok && lane == 0) {  // accumulator complete
          const uint32_t f = smem_u32(&bar_acc_full[buf]);
          if (PAIR) {
            tc_commit<true>(mapa(f, 0));
            tc_commit<true>(mapa(f, 1));
          } else {
            tc_commit<false>(f);
          }
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const uint32_t stage_addr = ((smem_u32(smem_raw) + 1023u) & ~1023u) + p.stage_off + (uint32_t)(warp - 2) * (uint32_t)(32 * p.out_row_bytes);
    const bool split = !p.batched && p.splits > 1;
#define OXB_EPI(V)                                                                                                                                    \
  case V:                                                                                                                                             \
    if (!PAIR && split) epilogue_role<BN, KIND, V, !PAIR, PAIR>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles, tile0, tile_step, pair_rank); \
    else epilogue_role<BN, KIND, V, false, PAIR>(p, warp, lane, tmem_base, bar_acc_full, bar_acc_empty, stage_addr, abortp, total_tiles, tile0, tile_step, pair_rank); \
    break;
    if constexpr (KIND == KIND_I8) {
      switch (p.variant) {
        OXB_EPI(V_REQUANT)
        OXB_EPI(V_REQUANT_DYN)
        OXB_EPI(V_INT32)
        OXB_EPI(V_INT32_DYN)
        OXB_EPI(V_REQUANT_FMA)
        OXB_EPI(V_REQUANT_FMA_DYN)
        OXB_EPI(V_REQUANT_LEAN)
        OXB_EPI(V_REQUANT_LEAN_DYN)
        OXB_EPI(V_REQUANT_FBIAS)
        OXB_EPI(V_REQUANT_PACKED)
        OXB_EPI(30)
        OXB_EPI(31)
        OXB_EPI(32)
        OXB_EPI(33)
        OXB_EPI(34)
        OXB_EPI(35)
        default: break;
      }
    } else {
      switch (p.variant) {
        OXB_EPI(0)
        OXB_EPI(1)
        OXB_EPI(2)
        OXB_EPI(3)
        OXB_EPI(4)
        OXB_EPI(5)
        OXB_EPI(6)
        OXB_EPI(7)
        OXB_EPI(8)
        OXB_EPI(9)
        OXB_EPI(10)
        OXB_EPI(11)
        OXB_EPI(12)
        OXB_EPI(13)
        OXB_EPI(14)
        OXB_EPI(15)
        OXB_EPI(16)
        OXB_EPI(17)
        OXB_EPI(18)
        OXB_EPI(19)
        default: break;
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
  if (PAIR) cluster_sync_all();  // neither CTA ends while the other may still signal into its shared memory
  if (warp == 1) {
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ES::TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ES::TMEM_COLS) : "memory");
  }
}

// ---- launch -----------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;


// Per kind (one translation unit each): dispatch on the tile width.
void launch_kind_i8(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s);
void launch_kind_tf32(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s);
void launch_kind_f16(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s);
// How many CTA pairs of the 256-wide kernel of this kind can be resident at once on `device`.
int max_pairs_kind_i8(size_t smem, int device);
int max_pairs_kind_tf32(size_t smem, int device);
int max_pairs_kind_f16(size_t smem, int device);

}  // namespace umma
}  // namespace k
}  // namespace oxb
