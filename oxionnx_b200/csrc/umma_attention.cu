// One attention layer's f32 side as one tcgen05 kernel: scores = Q K^T, probabilities = softmax(scores * scale +
// mask) over the last axis, context = probabilities . V, per (batch, head), for sequences of 128 positions and
// heads of 64 lanes (TF32 operands, f32 accumulation, as the two separate batched products use).
//
// The scores never leave the SM: the first product accumulates a 128 x 128 tile in TMEM, the accumulator warps'
// threads read it into registers (32 scores of a row each), applies the scalar product and the additive mask
// (each rounded as the separate Mul and Add nodes round), the row softmax (max, exp(v - max), an f32 sum, one
// reciprocal, one product per lane, nn/normalization.rs softmax_into) and the TF32 rounding of lanes that feed
// a contraction, and writes the row into shared memory in the 128-byte-swizzled K-major layout a TMA load would
// have left; the second product reads it from there.  Q and K are column windows of their [B * S, H * D]
// matrices, V arrives transposed per head ([B * H * D, S]), the context is stored by TMA straight into its (possibly
// head-merged) matrix.  One warp loads and issues; sixteen warps do the rows, four threads per row (32 scores each,
// the row's maximum and sum meet in shared memory behind two mbarriers); a CTA walks the (batch, head) items and
// loads the next item's operands as soon as the current product has read them.  Every wait is bounded.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "umma_kernel.cuh"

namespace oxb {
namespace k {

namespace umma {

constexpr int ATT_S = 128, ATT_D = 64;
constexpr int ATT_ROW_WARPS = 16;                      // warp w: accumulator rows 32 (w & 3) .. + 31, score columns 32 (w >> 2) .. + 31
constexpr int ATT_THREADS = 32 * ATT_ROW_WARPS + 32;   // plus one warp that loads and issues
constexpr uint32_t ATT_Q_OFF = 0, ATT_K_OFF = 32768, ATT_V_OFF = 65536, ATT_P_OFF = 98304, ATT_O_OFF = 163840;
constexpr uint32_t ATT_SMEM = 163840 + 32768 + 1024;   // Q, K, V^T, probabilities, context staging, alignment slack

struct alignas(64) AttnParams {
  CUtensorMap tmQ, tmK, tmV, tmO;
  int items, heads;
  uint32_t idesc_s, idesc_o;
  const float* scale;  // one device lane, or null
  const float* mask;   // [batch][128] additive, or null
  int o_rb, o_rh, o_ch;
  int round_probs;
  unsigned int* minmax_keys;
  int* err_flag;
};

__global__ void __launch_bounds__(ATT_THREADS, 1) umma_attention_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_qk, bar_v, bar_s, bar_p, bar_o, bar_max, bar_sum;
  __shared__ float row_max[4][ATT_S], row_sum[4][ATT_S];  // per column block of 32 scores
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int warp = (int)(threadIdx.x >> 5), lane = (int)(threadIdx.x & 31);
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  volatile int* abortp = &abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar_qk), 1);
    mbar_init(smem_u32(&bar_v), 1);
    mbar_init(smem_u32(&bar_s), 1);
    mbar_init(smem_u32(&bar_p), 32 * ATT_ROW_WARPS);
    mbar_init(smem_u32(&bar_o), 1);
    mbar_init(smem_u32(&bar_max), 32 * ATT_ROW_WARPS);
    mbar_init(smem_u32(&bar_sum), 32 * ATT_ROW_WARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == ATT_ROW_WARPS) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 128u;
  auto give_up = [&](int code) {
    if (!*abortp) {
      *abortp = 1;
      atomicExch(p.err_flag, code);
    }
  };

  if (warp == ATT_ROW_WARPS) {
    // ---------------- loads and MMA issue ----------------
    auto load_qk = [&](int item) {
      const int b = item / p.heads, h = item - b * p.heads;
      mbar_expect_tx(smem_u32(&bar_qk), 65536u);
      for (int kb = 0; kb < 2; ++kb) {
        tma_load_2d(base + ATT_Q_OFF + (uint32_t)kb * 16384u, &p.tmQ, smem_u32(&bar_qk), h * ATT_D + kb * 32, b * ATT_S);
        tma_load_2d(base + ATT_K_OFF + (uint32_t)kb * 16384u, &p.tmK, smem_u32(&bar_qk), h * ATT_D + kb * 32, b * ATT_S);
      }
    };
    auto load_v = [&](int item) {
      mbar_expect_tx(smem_u32(&bar_v), 32768u);
      for (int kb = 0; kb < 4; ++kb) tma_load_2d(base + ATT_V_OFF + (uint32_t)kb * 8192u, &p.tmV, smem_u32(&bar_v), kb * 32, item * ATT_D);
    };
    if (lane == 0 && (int)blockIdx.x < p.items) {
      load_qk((int)blockIdx.x);
      load_v((int)blockIdx.x);
    }
    __syncwarp();
    const uint64_t desc_rest = make_smem_desc(0, 128);
    const uint32_t desc_hi = (uint32_t)(desc_rest >> 32), desc_lo = (uint32_t)desc_rest;
    uint32_t phase = 0;
    for (int item = (int)blockIdx.x; item < p.items; item += (int)gridDim.x, phase ^= 1u) {
      const int next = item + (int)gridDim.x;
      bool got = mbar_wait(smem_u32(&bar_qk), phase, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(31);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        for (int kb = 0; kb < 2; ++kb)
          tc_mma_block<KIND_TF32, false>(tmem_s, desc_lo | (((base + ATT_Q_OFF + (uint32_t)kb * 16384u) >> 4) & 0x3fffu),
                                         desc_lo | (((base + ATT_K_OFF + (uint32_t)kb * 16384u) >> 4) & 0x3fffu), desc_hi, p.idesc_s, kb > 0 ? 1u : 0u, 4u);
        tc_commit<false>(smem_u32(&bar_s));
      }
      __syncwarp();
      got = mbar_wait(smem_u32(&bar_s), phase, abortp);  // Q and K have been read
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(32);
        break;
      }
      if (lane == 0 && next < p.items) load_qk(next);
      __syncwarp();
      got = mbar_wait(smem_u32(&bar_p), phase, abortp);  // the probabilities are in shared memory
      got = mbar_wait(smem_u32(&bar_v), phase, abortp) && got;
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(33);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        for (int kb = 0; kb < 4; ++kb)
          tc_mma_block<KIND_TF32, false>(tmem_o, desc_lo | (((base + ATT_P_OFF + (uint32_t)kb * 16384u) >> 4) & 0x3fffu),
                                         desc_lo | (((base + ATT_V_OFF + (uint32_t)kb * 8192u) >> 4) & 0x3fffu), desc_hi, p.idesc_o, kb > 0 ? 1u : 0u, 4u);
        tc_commit<false>(smem_u32(&bar_o));
      }
      __syncwarp();
      got = mbar_wait(smem_u32(&bar_o), phase, abortp);  // V and the probabilities have been read
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(34);
        break;
      }
      if (lane == 0 && next < p.items) load_v(next);
      __syncwarp();
    }
  } else {
    // ---------------- 32 scores of one row per thread; four threads share a row through shared memory ----------------
    const int quarter = warp & 3, cb = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sc = p.scale ? __ldg(p.scale) : 1.f;
    float seen_min = INFINITY, seen_max = -INFINITY;
    // context staging of this warp (the warps of column blocks 0 and 1 write the context): 32 rows x 128 bytes
    const uint32_t stage = base + ATT_O_OFF + (uint32_t)((cb & 1) * 4 + quarter) * 4096u;
    uint8_t* stage_ptr = base_ptr + ATT_O_OFF + ((cb & 1) * 4 + quarter) * 4096;
    uint32_t phase = 0;
    for (int item = (int)blockIdx.x; item < p.items; item += (int)gridDim.x, phase ^= 1u) {
      const int b = item / p.heads, h = item - b * p.heads;
      bool got = mbar_wait(smem_u32(&bar_s), phase, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(35);
        break;
      }
      tc_fence_after();
      float v[32];
      {
        uint32_t r[32];
        tmem_ld32_nowait(tmem_s + lane_base + (uint32_t)cb * 32u, r);
        tmem_ld_wait_for(r);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      }
      tc_fence_before();
      const float4* pm = p.mask ? reinterpret_cast<const float4*>(p.mask + (size_t)b * ATT_S + cb * 32) : nullptr;
      float mx = -INFINITY;
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
        if (pm) m = __ldg(pm + j4);
        const float mm[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = v[4 * j4 + e];
          if (p.scale) x = __fmul_rn(x, sc);
          if (pm) x = __fadd_rn(x, mm[e]);
          v[4 * j4 + e] = x;
          mx = fmaxf(mx, x);
        }
      }
      row_max[cb][row] = mx;
      mbar_arrive(smem_u32(&bar_max));
      got = mbar_wait(smem_u32(&bar_max), phase, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(36);
        break;
      }
      mx = fmaxf(fmaxf(row_max[0][row], row_max[1][row]), fmaxf(row_max[2][row], row_max[3][row]));
      // exp through ex2.approx (two units in the last place, far inside the softmax tolerance of 1e-5)
      float part[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = __expf(__fsub_rn(v[j], mx));
        part[j & 1] = __fadd_rn(part[j & 1], v[j]);
      }
      row_sum[cb][row] = __fadd_rn(part[0], part[1]);
      mbar_arrive(smem_u32(&bar_sum));
      got = mbar_wait(smem_u32(&bar_sum), phase, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(37);
        break;
      }
      const float inv = __frcp_rn(__fadd_rn(__fadd_rn(row_sum[0][row], row_sum[1][row]), __fadd_rn(row_sum[2][row], row_sum[3][row])));
      // this thread's 32 lanes are K block `cb` of the row: 16-byte piece c sits at row * 128 + ((c ^ (row & 7)) << 4)
      uint8_t* prow = base_ptr + ATT_P_OFF + cb * 16384 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[e] = __fmul_rn(v[4 * c + e], inv);
          if (p.round_probs) o[e] = round_tf32(o[e]);
        }
        *reinterpret_cast<float4*>(prow + ((c ^ (row & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the second product reads the rows through the async proxy
      mbar_arrive(smem_u32(&bar_p));
      got = mbar_wait(smem_u32(&bar_o), phase, abortp);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) give_up(38);
        break;
      }
      if (cb < 2) {
        // 32 context lanes of the row: staged (swizzled as the store's tensor map expects) and stored by TMA
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32_nowait(tmem_o + lane_base + (uint32_t)cb * 32u, r);
        tmem_ld_wait_for(r);
        tc_fence_before();
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the previous store has read the staging rows
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(stage_ptr + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
          if (p.minmax_keys) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              seen_min = fminf(seen_min, __uint_as_float(r[4 * c + e]));
              seen_max = fmaxf(seen_max, __uint_as_float(r[4 * c + e]));
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&p.tmO, stage, h * p.o_ch + cb * 32, b * p.o_rb + h * p.o_rh + quarter * 32);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (cb < 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (p.minmax_keys && cb < 2) {
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

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the CTA's shared memory goes away
    const long long start = clock64();
    while (clock64() - start < 2000000LL) {
    }
  }
  __syncthreads();
  if (warp == ATT_ROW_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot), "r"(256) : "memory");
}

}  // namespace umma

using namespace umma;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn attention_encoder() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)f;
    (void)cudaGetLastError();
  });
  return fn;
}

// kind::tf32 instruction descriptor: f32 accumulator, TF32 operands, both K-major, N / 8 and M / 16
uint32_t tf32_idesc(int n, int m) { return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

bool encode_f32_matrix(EncodeTiledFn enc, CUtensorMap* tm, const void* ptr, int64_t cols, int64_t rows, int box_rows) {
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

struct UmmaAttentionPlan {
  AttnParams ap;
  int grid = 0, device = 0;
  char desc[160];
};

UmmaAttentionPlan* umma_attention_create(const FusedAttention& a, std::string* why) {
  auto no = [&](const char* msg) -> UmmaAttentionPlan* {
    if (why) *why = msg;
    return nullptr;
  };
  EncodeTiledFn enc = attention_encoder();
  if (!enc) return no("tensor-map encoders unavailable in this driver");
  if (a.S != ATT_S || a.D != ATT_D) return no("only 128 positions x 64 lanes per head");
  if (a.B <= 0 || a.H <= 0 || (int64_t)a.B * a.H > 0x3fffffff) return no("empty or oversized problem");
  if (((uintptr_t)a.q & 127) || ((uintptr_t)a.k & 127) || ((uintptr_t)a.vt & 127) || ((uintptr_t)a.out & 15) || ((uintptr_t)a.mask & 15)) return no("operand base address is not aligned");
  if ((a.o_cols % 4) || (a.o_ch % 4)) return no("output columns are not 16-byte granular");
  UmmaAttentionPlan* pl = new UmmaAttentionPlan();
  std::memset(&pl->ap, 0, sizeof(AttnParams));
  AttnParams& ap = pl->ap;
  const int64_t rows = (int64_t)a.B * a.S, cols = (int64_t)a.H * a.D;
  if (!encode_f32_matrix(enc, &ap.tmQ, a.q, cols, rows, ATT_S) || !encode_f32_matrix(enc, &ap.tmK, a.k, cols, rows, ATT_S) ||
      !encode_f32_matrix(enc, &ap.tmV, a.vt, a.S, (int64_t)a.B * a.H * a.D, ATT_D)) {
    delete pl;
    return no("tensor map rejected by the driver");
  }
  ap.items = a.B * a.H;
  ap.heads = a.H;
  ap.idesc_s = tf32_idesc(ATT_S, 128);
  ap.idesc_o = tf32_idesc(ATT_D, 128);
  ap.scale = a.scale;
  ap.mask = a.mask;
  {
    // the context goes out by TMA: 32 rows x 32 lanes per store, out of 128-byte-swizzled staging rows
    cuuint64_t gdim[2] = {(cuuint64_t)a.o_cols, (cuuint64_t)a.o_rows};
    cuuint64_t gstr[1] = {(cuuint64_t)a.o_cols * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&ap.tmO, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, a.out, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      delete pl;
      return no("output tensor map rejected by the driver");
    }
  }
  ap.o_rb = a.o_rb, ap.o_rh = a.o_rh, ap.o_ch = a.o_ch;
  ap.round_probs = a.round_probs;
  ap.minmax_keys = a.minmax_keys;
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) (void)cudaGetLastError();
  pl->device = device;
  pl->grid = std::min(ap.items, sms);
  snprintf(pl->desc, sizeof pl->desc, "umma_attention %dx%d heads of 128x64: scores, softmax%s%s and context in one kernel, grid=%d", a.B, a.H, a.scale ? "+scale" : "",
           a.mask ? "+mask" : "", pl->grid);
  return pl;
}

void umma_attention_destroy(UmmaAttentionPlan* p) { delete p; }
const char* umma_attention_desc(const UmmaAttentionPlan* p) { return p->desc; }

void umma_attention_launch(const UmmaAttentionPlan* p, int* err_flag, cudaStream_t s) {
  // the opt-in for more than 48 KB of dynamic shared memory is a per-device property of the kernel
  static std::mutex mu;
  static bool have[kMaxDevices] = {};
  {
    std::lock_guard<std::mutex> lock(mu);
    const int d = (p->device >= 0 && p->device < kMaxDevices) ? p->device : 0;
    if (!have[d]) {
      OXB_CUDA(cudaFuncSetAttribute(umma_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_SMEM));
      have[d] = true;
    }
  }
  AttnParams ap = p->ap;
  ap.err_flag = err_flag;
  umma_attention_kernel<<<p->grid, ATT_THREADS, ATT_SMEM, s>>>(ap);
  OXB_CUDA(cudaGetLastError());
}

}  // namespace k
}  // namespace oxb
