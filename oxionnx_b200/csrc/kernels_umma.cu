// tcgen05 implicit-GEMM convolution / GEMM for sm_100a: plan creation (tile model, tensor maps, epilogue
// variant) and launch dispatch.  The device code lives in umma_kernel.cuh and is instantiated per kind in
// umma_i8.cu, umma_tf32.cu and umma_f16.cu.
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "umma_chain.cuh"
#include "umma_kernel.cuh"

namespace oxb {
namespace k {

using namespace umma;

namespace {

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

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return dev;
}

// Per device: a process may hold one context per GPU, on threads of its own.
int sm_count(int device) {
  static std::mutex mu;
  static int cached[kMaxDevices] = {};
  const int d = (device >= 0 && device < kMaxDevices) ? device : 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[d] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && n > 0) cached[d] = n;
    else cached[d] = 148;
    (void)cudaGetLastError();
  }
  return cached[d];
}

CUtensorMapSwizzle swizzle_enum(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

CUtensorMapDataType operand_map_type(int kind) {
  switch (kind) {
    case KIND_I8: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case KIND_TF32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case KIND_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  }
}

CUtensorMapDataType output_map_type(DT dt) {
  switch (dt) {
    case DT::F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case DT::I32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
    case DT::F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case DT::BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case DT::I16: return CU_TENSOR_MAP_DATA_TYPE_UINT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// Instruction descriptor: accumulator and operand formats, K-major operands, N / 8 and M / 16.
uint32_t make_idesc(int kind, bool a_signed, bool b_signed, int bn, int m) {
  uint32_t d = 0;
  if (kind == KIND_I8) {
    d |= 2u << 4;                      // accumulator: s32
    d |= (a_signed ? 1u : 0u) << 7;    // A: 0 = u8, 1 = s8
    d |= (b_signed ? 1u : 0u) << 10;   // B
  } else if (kind == KIND_TF32) {
    d |= 1u << 4;  // accumulator: f32
    d |= 2u << 7;  // A: tf32
    d |= 2u << 10; // B: tf32
  } else {
    d |= 1u << 4;                                   // accumulator: f32
    d |= (kind == KIND_BF16 ? 1u : 0u) << 7;        // A: 0 = f16, 1 = bf16
    d |= (kind == KIND_BF16 ? 1u : 0u) << 10;       // B
  }
  // bits 15/16: A and B are K-major (0)
  d |= (uint32_t)(bn >> 3) << 17;
  d |= (uint32_t)(m >> 4) << 24;
  return d;
}

// Shared memory of one CTA: 227 KB less the kernel's static part (barriers) and alignment slack.
constexpr size_t kSmemBudget = 227 * 1024 - 2048;

}  // namespace

struct UmmaPlan {
  KParams kp;
  int bn;
  int kind;
  int pair;
  int grid;
  int device;
  size_t smem;
  char desc[176];
  void* ws = nullptr;        // split-K workspace and arrival counters, owned by the plan
  void* ws_count = nullptr;
};

bool umma_available() {
  load_encoders();
  return g_encode_tiled != nullptr && g_encode_im2col != nullptr;
}

bool umma_overlapping_positions_ok() {
  static std::once_flag once;
  static bool ok = false;
  std::call_once(once, [] {
    load_encoders();
    if (!g_encode_im2col) return;
    // the shape of the 8-bit stem: 64-lane windows 16 lanes apart; nothing is read through this map
    CUtensorMap tm;
    cuuint64_t gdim[4] = {64, 112, 112, 2};
    cuuint64_t gstr[3] = {16, 115 * 16, 112 * 115 * 16};
    int lower[2] = {0, -2}, upper[2] = {0, -2};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult rc = g_encode_im2col(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, reinterpret_cast<void*>(uintptr_t(1) << 30), gdim, gstr, lower, upper, 64, BLOCK_M,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ok = rc == CUDA_SUCCESS;
  });
  return ok;
}

int umma_channel_block(int C, int kind) {
  const int es = umma_elem_bytes(kind);
  int64_t row = (int64_t)C * es;
  if (row % 128 == 0) return 128 / es;
  if (row == 64) return 64 / es;
  if (row == 32) return 32 / es;
  return 0;
}

namespace {

// Ring depth and the shared-memory layout [ring | epilogue staging rows] of a plan.
// Layout: [resident weights, when kp.b_resident_bytes > 0 | ring | staging rows].
void layout_smem(KParams& kp, int bn, int kind, bool pair, size_t* smem_total) {
  const int ew = epi_warps(kind);
  const size_t resident = kp.b_resident_bytes;
  const size_t kb_bytes = (size_t)(BLOCK_M + (resident ? 0 : (pair ? bn / 2 : bn))) * kp.swizzle_bytes;
  const size_t stage_bytes = kb_bytes * kp.kpb;
  const size_t staging = kp.out_tma ? (size_t)ew * 32 * kp.out_row_bytes : 0;
  // one persistent CTA per SM: the ring may use most of the shared memory and runs on across tiles
  const size_t budget = std::min<size_t>(192 * 1024, kSmemBudget - staging) - resident;
  int stages = (int)(budget / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) stages = 2;
  kp.stages = stages;
  kp.stage_off = (uint32_t)(resident + stages * stage_bytes);
  *smem_total = resident + (size_t)stages * stage_bytes + staging + 1024;
}

// Bytes of an output row one epilogue warp stages per TMA store: its share of the row, at most 128.
size_t warp_row_bytes(int bn, int kind, size_t oes, bool one_run) {
  const int ew = epi_warps(kind);
  const int runs = bn / 32, wpq_all = ew / 4;
  const int wpq = std::min(wpq_all, std::max(runs / 2, 1));  // EpiShape::WPQ
  const int cpw = one_run ? 1 : runs / wpq;
  return std::min<size_t>(128, (size_t)cpw * 32 * oes);
}

}  // namespace

UmmaPlan* umma_plan_create(const void* x, DT x_dt, const void* w_packed, DT w_dt, void* out, const ConvShape& cs, const Epilogue& e, int kind,
                           const UmmaTuning& tune, std::string* why) {
  auto no = [&](const char* msg) -> UmmaPlan* {
    if (why) *why = msg;
    return nullptr;
  };
  load_encoders();
  if (!g_encode_tiled || !g_encode_im2col) return no("tensor-map encoders unavailable in this driver");
  if (cs.group != 1) return no("grouped convolution");
  if (kind == KIND_I8) {
    if (!(x_dt == DT::U8 || x_dt == DT::I8) || !(w_dt == DT::I8 || w_dt == DT::U8)) return no("operands are not 8-bit integers");
    if (e.mode == EPI_F32) return no("integer kind needs an integer epilogue");
  } else if (kind == KIND_TF32) {
    if (x_dt != DT::F32 || w_dt != DT::F32 || e.mode != EPI_F32) return no("tf32 kind needs f32 operands and a float epilogue");
  } else {
    const DT want = kind == KIND_F16 ? DT::F16 : DT::BF16;
    if (x_dt != want || w_dt != want || e.mode != EPI_F32) return no("16-bit float kind needs matching 16-bit operands and a float epilogue");
  }
  const int es = umma_elem_bytes(kind);
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
  if (e.mode == EPI_F32 ? e.bias_f == nullptr : e.bias_i == nullptr) return no("the tensor-core epilogue needs a (padded) bias vector");
  if (e.mode == EPI_F32 && e.act == 4 && e.slope == nullptr) return no("the PRelu epilogue needs a (padded) slope vector");

  // Tile width.  Measured on B200 (1.965 GHz): a tcgen05.mma of 32 bytes of K takes N/2 cycles
  // of the tensor pipe but cannot be issued faster than one per ~56 cycles; one SM fills its
  // shared memory from L2 at about 95 GB/s when all SMs do so; the fused epilogue costs about
  // 0.07 ns per output for requantisation and 0.03 ns for the float variants, plus a fixed cost per tile.  The three overlap
  // (ring of stages, two accumulators), so a tile takes the longest of them, the kernel runs
  // ceil(tiles / SMs) rounds of tiles, and the last tile's epilogue is not hidden.  Pick the
  // width that minimises that estimate; ties go to the wider tile (fewer re-reads of the activations).
  // Split K: when even the narrowest useful tiling leaves most SMs without a tile and K is long, `splits`
  // CTAs share a (wider) tile, each running a slice of K; the slices meet in an L2-resident workspace.  It is
  // only considered when every slice gets its own SM in one round and at least eight K blocks.
  const int device = current_device();
  const int sms = sm_count(device);
  const int64_t m_tiles = ceil_div(M, BLOCK_M);
  const int bn_max = cs.OC <= 32 ? 32 : (cs.OC <= 64 ? 64 : (cs.OC <= 128 ? 128 : 256));
  const int64_t k_iters_host = (int64_t)cs.R * cs.S * (cs.C / cb);
  int bn = bn_max, splits = 1;
  {
    const double k_bytes = (double)cs.K() * es;
    const double k_steps = k_bytes / 32.0;
    // epilogue: per output 0.07 ns requantised / 0.03 ns float, plus about 0.5 us per tile whatever its width (the
    // per-tile handshakes and address arithmetic of the epilogue warps: a 1x1 64 -> 256 layer at M = 802816 takes
    // 3.0 us per round of 128 x 256 tiles, 1.05 us per round of 128 x 64 tiles, 0.84 us per round of 128 x 32)
    const double ns_out = e.mode == EPI_F32 ? 0.03e-9 : 0.07e-9;
    const double t_tile_fixed = 0.5e-6;
    const int max_split = tune.split_k_max > 0 ? tune.split_k_max : 8;
    double best = 1e30;
    for (int cand = bn_max; cand >= 32; cand /= 2) {
      const double tiles = (double)m_tiles * (double)ceil_div(cs.OC, cand);
      for (int sp = 1; sp <= max_split; ++sp) {
        if (sp > 1 && (tiles * sp > sms || k_iters_host / sp < 8)) break;
        const double rounds = std::ceil(tiles * sp / sms);
        const double t_mma = k_steps * std::max(56.0, cand / 2.0) / 1.965e9 / sp;
        const double t_feed = (double)(BLOCK_M + cand) * k_bytes / 95e9 / sp;
        const double t_epi = (double)BLOCK_M * cand * ns_out + t_tile_fixed;
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
  // CTA pairs: two CTAs share a 256 x 256 tile and each stages 128 rows of A and 128 rows of B per K block (32 KB
  // at 128-byte K blocks instead of the 48 KB of a lone CTA's 128 x 256 tile), which relieves both the L2 -> shared
  // memory feed and the shared-memory bandwidth the MMAs and the incoming copies compete for.  Worth it where the
  // operand feed bounds the tile (long K) and there are enough 256-row tiles to keep every pair busy.
  bool pair = false;
  if (tune.cta_pairs == 2 && cs.OC >= 256) {  // forced (tests, comparisons): the pair form wherever the shape allows it
    bn = 256;
    splits = 1;
  }
  if (tune.cta_pairs != 1 && bn == 256 && splits == 1 && cs.OC >= 256) {
    const int64_t pair_tiles = ceil_div(M, 2 * BLOCK_M) * ceil_div(cs.OC, 256);
    const double k_bytes = (double)cs.K() * es;
    // Measured: with 2 KB of K or more per row a pair wins once every pair has at least two tiles (3x3 256->256,
    // i8, M=100352: 57.7 us against 65.9 us for lone CTAs); from 8 KB of K it also wins with a single partial wave
    // (TF32 3x3 256->256 at M=25088: 61.9 us against 78.2 us); below 2 KB the extra barrier traffic of a pair costs
    // more than the halved operand feed saves (1x1 1024->256, i8, M=12544: 18.6 us against 16.7 us).
    const int64_t pairs_resident = sms / 2;
    const bool feed_bound = k_bytes >= 2048.0 && (pair_tiles >= 2 * pairs_resident || (k_bytes >= 8192.0 && pair_tiles >= pairs_resident));
    if (tune.cta_pairs == 2) pair = true;
    else pair = feed_bound;
  }
  const int64_t n_tiles = ceil_div(cs.OC, bn);
  if (m_tiles * n_tiles > 0x7fffffffLL) return no("grid too large");

  UmmaPlan* pl = new UmmaPlan();
  std::memset(&pl->kp, 0, sizeof(KParams));
  KParams& kp = pl->kp;
  auto fail = [&](const char* msg) -> UmmaPlan* {
    if (pl->ws) cudaFree(pl->ws);
    if (pl->ws_count) cudaFree(pl->ws_count);
    delete pl;
    return no(msg);
  };
  const CUtensorMapDataType dtype = operand_map_type(kind);
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
  if (rc != CUDA_SUCCESS) return fail("activation tensor map rejected by the driver");
  {
    const int64_t ktot = cs.K();
    cuuint64_t gdim[2] = {(cuuint64_t)ktot, (cuuint64_t)cs.OC};
    cuuint64_t gstr[1] = {(cuuint64_t)ktot * es};
    cuuint32_t box[2] = {(cuuint32_t)cb, (cuuint32_t)(pair ? bn / 2 : bn)};  // a CTA of a pair stages its half of the channel tile
    cuuint32_t estr[2] = {1, 1};
    rc = g_encode_tiled(&kp.tmB, dtype, 2, const_cast<void*>(w_packed), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swz),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail("weight tensor map rejected by the driver");
  }
  {
    // output tile store through TMA when rows are 16-byte granular
    const size_t oes = dt_size(e.out_dt);
    // one epilogue warp's share of a row; one run when K is split (any slice may finish any run)
    const size_t row_bytes = warp_row_bytes(bn, kind, oes, splits > 1);
    kp.out_tma = 0;
    kp.out_row_bytes = (int)row_bytes;
    if (((size_t)cs.OC * oes) % 16 == 0 && ((uintptr_t)out & 15) == 0 && row_bytes >= 32 && (row_bytes & (row_bytes - 1)) == 0) {
      cuuint64_t gdim[2] = {(cuuint64_t)cs.OC, (cuuint64_t)M};
      cuuint64_t gstr[1] = {(cuuint64_t)cs.OC * oes};
      cuuint32_t box[2] = {(cuuint32_t)(row_bytes / oes), 32};
      cuuint32_t estr[2] = {1, 1};
      CUresult ro = g_encode_tiled(&kp.tmO, output_map_type(e.out_dt), 2, out, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle_enum((int)row_bytes), CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (ro == CUDA_SUCCESS) kp.out_tma = 1;
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
  kp.m_tiles = pair ? (int)ceil_div(M, 2 * BLOCK_M) : (int)m_tiles;
  kp.idesc = make_idesc(kind, x_dt == DT::I8, w_dt == DT::I8, bn, pair ? 2 * BLOCK_M : BLOCK_M);
  // K blocks per stage: up to four small ones share a barrier round trip, as long as a stage stays
  // within 64 KB (the ring then still has three stages)
  // A layer with one channel tile whose packed weights fit beside the ring keeps them in shared memory for the
  // life of the CTA: every tile after a CTA's first then fetches activation rows only.
  {
    const size_t b_total = (size_t)k_iters_host * bn * swz;
    // Measured (i8, M=802816): 3x3 64->64 125.1 us against 137.6 us, 1x1 256->64 53.6 against 55.6, 1x1 256->128 215.4 against 221.6.
    if (!pair && splits == 1 && n_tiles == 1 && b_total <= 48 * 1024 && m_tiles >= 2 * sms) kp.b_resident_bytes = (uint32_t)b_total;
  }
  const size_t kb_bytes = (size_t)(BLOCK_M + (kp.b_resident_bytes ? 0 : (pair ? bn / 2 : bn))) * swz;
  int kpb = 1;
  while (kpb < 4 && (size_t)(kpb * 2) * kb_bytes <= 64 * 1024 && kpb * 2 <= k_iters_host) kpb *= 2;
  kp.kpb = kpb;
  // slices of K: whole stages each, none empty
  kp.splits = 1;
  kp.k_per = (int)k_iters_host;
  if (splits > 1) {
    const int64_t k_per = ceil_div(ceil_div(k_iters_host, (int64_t)splits), (int64_t)kpb) * kpb;
    const int64_t eff = ceil_div(k_iters_host, k_per);
    bool have_ws = false;
    if (eff > 1) {
      const size_t ws_words = (size_t)m_tiles * n_tiles * eff * BLOCK_M * bn;
      const size_t cnt = (size_t)m_tiles * n_tiles * epi_warps(kind) * 4;
      if (cudaMalloc(&pl->ws, ws_words * 4) == cudaSuccess && cudaMalloc(&pl->ws_count, cnt * sizeof(unsigned int)) == cudaSuccess &&
          cudaMemset(pl->ws_count, 0, cnt * sizeof(unsigned int)) == cudaSuccess) {
        kp.splits = (int)eff;
        kp.k_per = (int)k_per;
        kp.ws = (uint32_t*)pl->ws;
        kp.ws_count = (unsigned int*)pl->ws_count;
        have_ws = true;
      } else {
        (void)cudaGetLastError();  // no workspace: run unsplit
      }
    }
    // the staged row was sized for one run per store; the unsplit loop stores a warp's whole share at once
    if (!have_ws && kp.out_tma && (int)warp_row_bytes(bn, kind, dt_size(e.out_dt), false) != kp.out_row_bytes) kp.out_tma = 0;
  }
  layout_smem(kp, bn, kind, pair, &pl->smem);
  kp.mode = e.mode;
  if (e.mode == EPI_F32) kp.variant = (e.residual ? V_F32_RES : V_F32_BASE) + e.act * 2 + (e.round_tf32 ? 1 : 0);
  else if (e.mode == EPI_REQUANT) {
    const bool fma = e.combined_fma_ok && tune.requant_f64 != 1;
    const bool lean = fma && e.acc_abs_bound > 0 && e.acc_abs_bound < 16777216;
    // packed saturation: 8-bit lanes, every result provably inside int16 (margin for the rounding and the clamp bounds)
    const bool packed = lean && e.bias_if && tune.requant_f64 == 0 && dt_size(e.out_dt) == 1 && e.q_abs_bound > 0 && e.q_abs_bound < 32000.0;
    if (e.x_zp_dev) kp.variant = lean ? V_REQUANT_LEAN_DYN : (fma ? V_REQUANT_FMA_DYN : V_REQUANT_DYN);
    else kp.variant = lean ? (packed ? V_REQUANT_PACKED : (e.bias_if ? V_REQUANT_FBIAS : V_REQUANT_LEAN)) : (fma ? V_REQUANT_FMA : V_REQUANT);
  }
  else if (e.mode == EPI_DEQUANT) kp.variant = V_DEQUANT + (e.x_zp_dev ? 1 : 0) + 2 * e.dq_act;
  else kp.variant = e.x_zp_dev ? V_INT32_DYN : V_INT32;
  kp.bias_f = e.bias_f;
  kp.slope = e.slope;
  kp.residual = e.residual;
  kp.dq_w_scale = e.dq_w_scale;
  kp.dq_x_scale = e.dq_x_scale_dev;
  kp.dq_bias = e.dq_bias;
  kp.act = e.act;
  kp.clip_lo = e.clip_lo;
  kp.clip_hi = e.clip_hi;
  kp.round_tf32 = e.round_tf32;
  kp.bias_i = e.bias_i;
  kp.bias_if = e.bias_if;
  kp.wsum = e.x_zp_dev ? e.wsum : nullptr;
  kp.x_zp_dev = e.x_zp_dev;
  kp.combined = e.combined;
  kp.y_zp = e.y_zp;
  kp.lo = (e.relu_fused && e.lo < 0) ? 0 : e.lo;
  kp.hi = e.hi;
  kp.out_dt = (int)e.out_dt;
  kp.out = out;
  kp.minmax_keys = e.out_dt == DT::F32 ? e.minmax_keys : nullptr;
  kp.err_flag = nullptr;
  pl->bn = bn;
  pl->kind = kind;
  pl->device = device;
  pl->pair = pair ? 1 : 0;
  if (pair) {
    // as many pairs as the device can hold at once (an odd SM of a cluster-scheduling group stays idle)
    int max_pairs = 0;
    try {
      max_pairs = kind == KIND_I8 ? max_pairs_kind_i8(pl->smem, device) : (kind == KIND_TF32 ? max_pairs_kind_tf32(pl->smem, device) : max_pairs_kind_f16(pl->smem, device));
    } catch (...) {
      max_pairs = 0;
    }
    if (max_pairs <= 0) return fail("the device cannot hold a CTA pair of this kernel");
    const int64_t pair_tiles = (int64_t)kp.m_tiles * kp.n_tiles;
    pl->grid = 2 * (int)std::min<int64_t>(pair_tiles, max_pairs);
  } else {
    pl->grid = (int)std::min<int64_t>(m_tiles * n_tiles * kp.splits, sms);
  }
  const char* kname = kind == KIND_I8 ? "i8" : (kind == KIND_TF32 ? "tf32" : (kind == KIND_F16 ? "f16" : "bf16"));
  char split_note[24] = "";
  if (kp.splits > 1) snprintf(split_note, sizeof split_note, " splitK=%d", kp.splits);
  snprintf(pl->desc, sizeof pl->desc, "umma_%s M=%lld N=%d K=%lld tile=%dx%dx%dB stages=%dx%d %s%s%s", kname, (long long)M, cs.OC, (long long)cs.K(),
           pair ? 256 : 128, bn, swz, kp.stages, kpb, gemm_like ? "tiled" : "im2col", split_note, pair ? " cta-pair" : "");
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
  const int cb = umma_channel_block(g.K, KIND_TF32);
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
    const size_t row_bytes = warp_row_bytes(bn, KIND_TF32, 4, false);
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
  kp.idesc = make_idesc(KIND_TF32, false, false, bn, BLOCK_M);
  const size_t kb_bytes = (size_t)(BLOCK_M + bn) * swz;
  int kpb = 1;
  while (kpb < 4 && (size_t)(kpb * 2) * kb_bytes <= 64 * 1024 && kpb * 2 <= kp.cblocks) kpb *= 2;
  kp.kpb = kpb;
  layout_smem(kp, bn, KIND_TF32, false, &pl->smem);
  kp.mode = EPI_F32;
  kp.variant = g.round_tf32 ? 1 : 0;
  kp.bias_f = g.zero_bias;
  kp.round_tf32 = g.round_tf32;
  kp.out_dt = (int)DT::F32;
  kp.out = g.out;
  kp.minmax_keys = g.minmax_keys;
  pl->bn = bn;
  pl->kind = KIND_TF32;
  pl->pair = 0;
  pl->device = current_device();
  pl->grid = (int)std::min<int64_t>(items * m_tiles * n_tiles, sm_count(pl->device));
  snprintf(pl->desc, sizeof pl->desc, "umma_tf32 batched %lldx(M=%d N=%d K=%d) tile=128x%dx%dB stages=%dx%d", (long long)items, g.M, g.N, g.K, bn, swz, kp.stages, kpb);
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
  const size_t cnt = (size_t)p->kp.m_tiles * p->kp.n_tiles * epi_warps(p->kind) * 4;
  (void)cudaMemset(p->ws_count, 0, cnt * sizeof(unsigned int));
}
const char* umma_plan_desc(const UmmaPlan* p) { return p->desc; }

// ---- chain of quantised linear layers over few rows ------------------------------------------------------------
struct UmmaChain {
  ChainParams cp;
  int grid = 0, device = 0;
  size_t smem = 0;
  void* w_tiles[CHAIN_MAX_LAYERS] = {nullptr, nullptr, nullptr, nullptr};  // the layers' weights in tile order, owned by the chain
  void* scratch = nullptr;  // partial sums of every unit, arrival counters (zero between launches), the grid barrier's counter
  size_t scratch_bytes = 0;
  char desc[288];
};

namespace {

// Units, shared-memory regions and grid of a chain; `cluster` > 1: the K slices of a channel tile are the CTAs of
// one cluster of that size, 1: as many slices per tile as keep every unit on its own SM, summed through L2.
bool chain_layout(UmmaChain* c, const UmmaChainLayer* layers, int n_layers, int sms, int cluster, const char** why) {
  ChainParams& cp = c->cp;
  cp.cluster = cluster;
  int grid = 0, kb_max = 0;
  for (int l = 0; l < n_layers; ++l) {
    ChainLayerParams& P = cp.layer[l];
    const int kblocks = layers[l].K / 128;
    P.N = layers[l].N;
    P.n_tiles = (int)ceil_div(layers[l].N, 128);
    int splits = 1;
    if (cluster > 1) {
      if (kblocks % cluster != 0 || P.n_tiles * cluster > sms) return *why = "the K blocks do not divide among the CTAs of a cluster", false;
      splits = cluster;
    } else {
      if (P.n_tiles > sms) return *why = "more channel tiles than SMs", false;
      for (int sp = 1; sp <= kblocks; ++sp)
        if (kblocks % sp == 0 && P.n_tiles * sp <= sms) splits = sp;
    }
    P.splits = splits;
    P.kb = kblocks / splits;
    grid = std::max(grid, P.n_tiles * splits);
    kb_max = std::max(kb_max, P.kb);
  }
  // shared memory: [weight regions | activation blocks].  A layer whose slice does not fit beside the earlier
  // ones takes over the region of an earlier layer once that layer's MMAs have completed.  In a cluster the
  // activation blocks also hold the CTA's partial sums (128 channels x 64 rows of int32) once the MMAs are done.
  const size_t x_bytes = std::max<size_t>((size_t)kb_max * CHAIN_X_TILE, cluster > 1 ? (size_t)CHAIN_ROWS * 128 * 4 : 0);
  if (x_bytes + 1024 >= kSmemBudget) return *why = "activation blocks exceed shared memory", false;
  const size_t w_budget = kSmemBudget - 1024 - x_bytes;
  size_t cursor = 0;
  int taken_by[CHAIN_MAX_LAYERS] = {-1, -1, -1, -1};
  for (int l = 0; l < n_layers; ++l) {
    ChainLayerParams& P = cp.layer[l];
    const size_t need = (size_t)P.kb * CHAIN_W_TILE;
    if (cursor + need <= w_budget) {
      P.w_off = (uint32_t)cursor;
      P.w_after = -1;
      cursor += need;
      continue;
    }
    int from = -1;
    for (int j = 0; j < l && from < 0; ++j)
      if (taken_by[j] < 0 && cp.layer[j].w_after < 0 && (size_t)cp.layer[j].kb * CHAIN_W_TILE >= need) from = j;
    if (from < 0) return *why = "weight slices do not fit in shared memory", false;
    taken_by[from] = l;
    P.w_off = cp.layer[from].w_off;
    P.w_after = from;
  }
  cp.x_off = (uint32_t)cursor;
  c->smem = cursor + x_bytes + 1024;
  c->grid = grid;
  if (chain_max_resident(c->smem, c->device, cluster) < grid) return *why = "the grid cannot be resident at once", false;
  return true;
}

}  // namespace

void umma_chain_destroy(UmmaChain* c);

UmmaChain* umma_chain_create(const UmmaChainLayer* layers, int n_layers, int rows, const UmmaChainEnds& ends, std::string* why) {
  auto no = [&](const char* msg) -> UmmaChain* {
    if (why) *why = msg;
    return nullptr;
  };
  load_encoders();
  if (!g_encode_tiled) return no("no tensor-map encoder");
  if (n_layers < 2 || n_layers > CHAIN_MAX_LAYERS) return no("a chain has 2 to 4 layers");
  if (rows < 1 || rows > CHAIN_ROWS) return no("a chain runs at most 64 rows");
  int device = 0, sms = 0;
  OXB_CUDA(cudaGetDevice(&device));
  OXB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  for (int l = 0; l < n_layers; ++l) {
    const UmmaChainLayer& L = layers[l];
    if (L.K % 128 != 0 || L.K < 128 || L.N < 1) return no("K is not a multiple of 128 bytes");
    if (((uintptr_t)L.x & 15) || ((uintptr_t)L.w & 15)) return no("operand not 16-byte aligned");
    if (l > 0 && (L.x != layers[l - 1].out || L.K != layers[l - 1].N)) return no("layers are not chained");
    if (dt_size(L.x_dt) != 1 || dt_size(L.w_dt) != 1) return no("operands are not 8-bit");
  }
  UmmaChain* c = new UmmaChain();
  std::memset(&c->cp, 0, sizeof(ChainParams));
  ChainParams& cp = c->cp;
  cp.n_layers = n_layers;
  cp.rows = rows;
  c->device = device;
  if (ends.head_x && ((uintptr_t)ends.head_x & 15) == 0) {
    cp.head_x = ends.head_x;
    cp.head_q = (uint8_t*)const_cast<void*>(layers[0].x);
    cp.head_k = layers[0].K;
    cp.head_scale = ends.head_scale, cp.head_zp = ends.head_zp, cp.head_lo = ends.head_lo, cp.head_hi = ends.head_hi;
  }
  if (ends.tail_out) {
    cp.tail_out = ends.tail_out;
    cp.tail_scale = ends.tail_scale, cp.tail_zp = ends.tail_zp, cp.tail_signed = ends.tail_signed;
  }
  // Clusters of 4, then 8, then 2 CTAs (partial sums meet in distributed shared memory); a cluster launch that
  // the driver refuses, or K blocks that do not divide, leave the L2 workspace form.
  const char* msg = "";
  bool laid = false;
  uint64_t* probe_bar = nullptr;
  for (int cluster : {4, 8, 2, 1}) {
    const char* m2 = "";
    if (!chain_layout(c, layers, n_layers, sms, cluster, &m2)) {
      if (cluster == 1) msg = m2;
      continue;
    }
    if (cluster > 1) {
      // one empty launch with this geometry: cooperative and cluster attributes together
      if (!probe_bar && (cudaMalloc(&probe_bar, 256) != cudaSuccess || cudaMemset(probe_bar, 0, 256) != cudaSuccess)) {
        (void)cudaGetLastError();
        continue;
      }
      ChainParams trial;
      std::memset(&trial, 0, sizeof trial);
      trial.cluster = cluster;
      trial.grid_bar = (unsigned long long*)probe_bar;
      trial.err_flag = (int*)(probe_bar + 8);
      const int grid = (c->grid + cluster - 1) / cluster * cluster;
      if (!try_launch_chain(trial, grid, c->smem, device, cluster)) continue;
      c->grid = grid;
    }
    laid = true;
    break;
  }
  if (probe_bar) cudaFree(probe_bar);
  if (!laid) {
    delete c;
    return no(msg[0] ? msg : "no geometry fits");
  }
  // scratch: per layer the partial sums of every unit (L2 workspace form) and n_tiles arrival counters, then the barrier counter
  size_t off = 0;
  size_t acc_off[CHAIN_MAX_LAYERS], cnt_off[CHAIN_MAX_LAYERS];
  for (int l = 0; l < n_layers; ++l) {
    acc_off[l] = off;
    if (cp.cluster == 1) off += (size_t)cp.layer[l].n_tiles * cp.layer[l].splits * CHAIN_ROWS * 128 * 4;
    cnt_off[l] = off;
    off += align_up((size_t)cp.layer[l].n_tiles * 4, 256);
  }
  const size_t bar_off = off;
  off += 256;
  if (cudaMalloc(&c->scratch, off) != cudaSuccess || cudaMemset(c->scratch, 0, off) != cudaSuccess) {
    (void)cudaGetLastError();
    if (c->scratch) cudaFree(c->scratch);
    delete c;
    return no("no memory for the partial sums");
  }
  c->scratch_bytes = off;
  cp.grid_bar = (unsigned long long*)((uint8_t*)c->scratch + bar_off);
  for (int l = 0; l < n_layers; ++l) {
    const UmmaChainLayer& L = layers[l];
    ChainLayerParams& P = cp.layer[l];
    cuuint32_t estr[2] = {1, 1};
    const size_t w_rows = (size_t)P.n_tiles * (L.K / 128) * 128;  // rows of 128 bytes
    CUresult rc = CUDA_ERROR_OUT_OF_MEMORY;
    if (cudaMalloc(&c->w_tiles[l], w_rows * 128) == cudaSuccess) {
      chain_repack(L.w, c->w_tiles[l], L.N, L.K, nullptr);
      if (cudaStreamSynchronize(nullptr) == cudaSuccess) {
        cuuint64_t wdim[2] = {128, (cuuint64_t)w_rows}, wstr[1] = {128};
        cuuint32_t wbox[2] = {128, 128};
        rc = g_encode_tiled(&P.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, c->w_tiles[l], wdim, wstr, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      }
    }
    (void)cudaGetLastError();
    cuuint64_t xdim[2] = {(cuuint64_t)L.K, (cuuint64_t)rows}, xstr[1] = {(cuuint64_t)L.K};
    cuuint32_t xbox[2] = {128, (cuuint32_t)CHAIN_ROWS};
    if (rc == CUDA_SUCCESS)
      rc = g_encode_tiled(&P.tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(L.x), xdim, xstr, xbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      umma_chain_destroy(c);
      return no("no memory for the repacked weights, or tensor map rejected by the driver");
    }
    // the weights are the 128-row operand (A), the activation rows the 64 columns (B)
    P.idesc = make_idesc(KIND_I8, L.w_dt == DT::I8, L.x_dt == DT::I8, CHAIN_ROWS, 128);
    P.bias_i = L.bias_i;
    P.combined = L.combined;
    P.y_zp = L.y_zp;
    P.lo = L.lo;
    P.hi = L.hi;
    P.out = (uint8_t*)L.out;
    P.ws = (int32_t*)((uint8_t*)c->scratch + acc_off[l]);
    P.fma_exact = L.fma_exact;
    P.tile_count = (unsigned int*)((uint8_t*)c->scratch + cnt_off[l]);
  }
  int n = snprintf(c->desc, sizeof c->desc, "umma_i8_chain rows=%d", rows);
  for (int l = 0; l < n_layers && n < (int)sizeof c->desc; ++l)
    n += snprintf(c->desc + n, sizeof c->desc - n, " %dx%d:%dt*%ds", layers[l].K, layers[l].N, cp.layer[l].n_tiles, cp.layer[l].splits);
  if (n < (int)sizeof c->desc)
    snprintf(c->desc + n, sizeof c->desc - n, " grid=%d %s smem=%zuK%s%s", c->grid, cp.cluster > 1 ? "clusters (distributed shared memory)" : "slices through L2",
             c->smem / 1024, cp.head_x ? " +quantize" : "", cp.tail_out ? " +dequantize" : "");
  return c;
}

void umma_chain_destroy(UmmaChain* c) {
  if (!c) return;
  for (void* w : c->w_tiles)
    if (w) cudaFree(w);
  if (c->scratch) cudaFree(c->scratch);
  delete c;
}
void umma_chain_reset_after_error(UmmaChain* c) {
  if (c && c->scratch) (void)cudaMemset(c->scratch, 0, c->scratch_bytes);
}
const char* umma_chain_desc(const UmmaChain* c) { return c->desc; }
bool umma_chain_launch(const UmmaChain* c, int* err_flag, const float* head_x, cudaStream_t s) {
  ChainParams cp = c->cp;
  cp.err_flag = err_flag;
  if (cp.head_x) {
    if (!head_x || ((uintptr_t)head_x & 15)) return false;
    cp.head_x = head_x;
  }
  return launch_chain(cp, c->grid, c->smem, c->device, cp.cluster, s);
}

void umma_launch(const UmmaPlan* p, int* err_flag, cudaStream_t s) {
  KParams kp = p->kp;
  kp.err_flag = err_flag;
  if (p->kind == KIND_I8) launch_kind_i8(kp, p->bn, p->pair != 0, p->grid, p->smem, p->device, s);
  else if (p->kind == KIND_TF32) launch_kind_tf32(kp, p->bn, p->pair != 0, p->grid, p->smem, p->device, s);
  else launch_kind_f16(kp, p->bn, p->pair != 0, p->grid, p->smem, p->device, s);
  OXB_CUDA(cudaGetLastError());
}

}  // namespace k
}  // namespace oxb
