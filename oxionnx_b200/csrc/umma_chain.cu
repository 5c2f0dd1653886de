// The cooperative kernel that runs a whole chain of quantised linear layers over at most 64 rows (see
// umma_chain.cuh for the scheme).  Every wait is bounded: a barrier that does not flip within WAIT_CYCLES makes
// the CTA record an error code, stop issuing work and leave through the common teardown.
#include <algorithm>
#include <mutex>

#include "umma_chain.cuh"
#include "umma_kernel.cuh"

namespace oxb {
namespace k {
namespace umma {

namespace {

// The grid-wide barrier is one 64-bit counter that only grows: every CTA adds one per barrier, and barrier k of a
// launch is passed once the counter has reached base + (k + 1) * n_ctas, where base is the counter's value at the
// launch rounded down to a multiple of n_ctas (a CTA that reads it late may see arrivals at barrier 0 of CTAs that
// started earlier, but never a full round: nobody passes barrier 0 without it).  One fence, one reduction and an
// acquire-poll per barrier; nothing to reset between launches or graph replays.
__device__ __forceinline__ unsigned long long ld_acquire_gpu64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool grid_barrier(unsigned long long* bar, unsigned long long target, volatile int* abort_flag) {
  __threadfence();
  atomicAdd(bar, 1ull);
  if (ld_acquire_gpu64(bar) >= target) return true;
  const long long start = clock64();
  while (ld_acquire_gpu64(bar) < target)
    if (*abort_flag || clock64() - start > WAIT_CYCLES) return false;
  return true;
}

__device__ __forceinline__ int4 ld_dsmem_v4(uint32_t cluster_addr) {
  int4 v;
  asm volatile("ld.shared::cluster.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(cluster_addr) : "memory");
  return v;
}

// units of a layer when the K slices of a tile are the CTAs of a cluster
__device__ __forceinline__ int cluster_units(const ChainLayerParams& L, int cluster) { return L.n_tiles * cluster; }

// ONNX requantisation of one channel.  fast(): where the host has proven the one-FMA form exact for this layer's
// scales and the accumulator is below 2^24 (so that its conversion is exact), s = fma(acc, c, 1.5 * 2^23 + zp)
// rounds acc * c + zp once to the integer grid, ties to even, and the result is the low byte of s after the clamp;
// it reports accumulators it cannot take.  exact(): the reference's own operations (one f64 product, one f64 sum,
// round half to even, saturate); f64 instructions are slow on this part, so they only run where fast() declined.
__device__ __noinline__ uint8_t requant_f64(int32_t a, float comb, int y_zp, int lo, int hi) {
  return (uint8_t)min(max(__double2int_rn(__dadd_rn(__dmul_rn((double)a, (double)comb), (double)y_zp)), lo), hi);
}
struct Requant {
  int32_t bias;
  float comb, magic_zp, flo, fhi;
  int y_zp, lo, hi, fma_exact;
  __device__ __forceinline__ void load(const ChainLayerParams& L, int ch) {
    bias = __ldg(L.bias_i + ch);
    comb = __ldg(L.combined + ch);
    magic_zp = 12582912.0f + (float)L.y_zp, flo = 12582912.0f + (float)L.lo, fhi = 12582912.0f + (float)L.hi;
    y_zp = L.y_zp, lo = L.lo, hi = L.hi, fma_exact = L.fma_exact;
  }
  __device__ __forceinline__ uint8_t fast(uint32_t raw, bool& declined) const {
    const int32_t a = (int32_t)raw + bias;
    declined = declined || !fma_exact || a <= -16777216 || a >= 16777216;
    return (uint8_t)(__float_as_uint(fminf(fmaxf(fmaf(__int2float_rn(a), comb, magic_zp), flo), fhi)) & 0xffu);
  }
  __device__ __forceinline__ uint8_t exact(uint32_t raw) const { return requant_f64((int32_t)raw + bias, comb, y_zp, lo, hi); }
};

__device__ __forceinline__ void fail(volatile int* abort_flag, int* err_flag, int code) {
  if (!*abort_flag) {
    *abort_flag = 1;
    atomicExch(err_flag, code);
  }
}

}  // namespace

__global__ void __launch_bounds__(CHAIN_THREADS, 1) umma_chain_kernel(const __grid_constant__ ChainParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_w[CHAIN_MAX_LAYERS];  // a layer's weight slice has landed (each used once)
  __shared__ __align__(8) uint64_t bar_x;                    // the activation blocks of the current layer have landed
  __shared__ __align__(8) uint64_t bar_mma;                  // the current layer's MMAs have completed
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ unsigned int last_slot;

  const int warp = (int)(threadIdx.x >> 5), lane = (int)(threadIdx.x & 31);
  const int cta = (int)blockIdx.x;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int l = 0; l < CHAIN_MAX_LAYERS; ++l) mbar_init(smem_u32(&bar_w[l]), 1);
    mbar_init(smem_u32(&bar_x), 1);
    mbar_init(smem_u32(&bar_mma), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(CHAIN_ROWS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // the weight slice of layer l for this CTA: kb blocks of [128 channels x 128 bytes of K]
  auto issue_weights = [&](int l) {
    const ChainLayerParams& L = p.layer[l];
    if (cta >= L.n_tiles * L.splits) return;
    const int tile = cta / L.splits, slice = cta % L.splits;
    const uint32_t bar = smem_u32(&bar_w[l]);
    mbar_expect_tx(bar, (uint32_t)L.kb * CHAIN_W_TILE);
    // the weights were repacked tile by tile: K block b of channel tile t is rows [(t * kblocks + b) * 128, +128) of a
    // matrix of 128-byte rows, 16 KB contiguous in HBM
    const int kblocks = L.kb * L.splits;
    for (int i = 0; i < L.kb; ++i)
      tma_load_2d(base + L.w_off + (uint32_t)i * CHAIN_W_TILE, &L.tmW, bar, 0, (tile * kblocks + slice * L.kb + i) * 128);
  };
  if (warp == 4 && lane == 0)
    for (int l = 0; l < p.n_layers; ++l)
      if (p.layer[l].w_after < 0) issue_weights(l);

  const bool clustered = p.cluster > 1;
  int4* dump = reinterpret_cast<int4*>(smem_raw + (base - smem_u32(smem_raw)) + p.x_off);
  unsigned long long bar_base = 0;
  if (threadIdx.x == 0) {
    bar_base = ld_acquire_gpu64(p.grid_bar);
    bar_base -= bar_base % gridDim.x;
  }
  // A QuantizeLinear in front of the chain: the grid quantises the f32 rows once, 16 lanes per thread, into the
  // first layer's 8-bit rows (q = clamp(rint(x / scale) + zp)), and meets at the grid barrier before anybody loads
  // them; the weight loads issued above are in flight meanwhile.
  unsigned int barriers_done = 0;
  if (p.head_x != nullptr) {
    if (warp < 4) {
      const int64_t pieces = (int64_t)p.rows * p.head_k / 16;
      for (int64_t i = (int64_t)cta * 128 + threadIdx.x; i < pieces; i += (int64_t)gridDim.x * 128) {
        const float4* src = reinterpret_cast<const float4*>(p.head_x) + i * 4;
        uint32_t packed[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float4 v = __ldg(src + g);
          const float f[4] = {v.x, v.y, v.z, v.w};
          packed[g] = 0u;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float q = fminf(fmaxf(__fadd_rn(rintf(__fdiv_rn(f[e], p.head_scale)), p.head_zp), p.head_lo), p.head_hi);
            packed[g] |= ((uint32_t)__float2int_rn(q) & 0xffu) << (8 * e);
          }
        }
        reinterpret_cast<uint4*>(p.head_q)[i] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && !grid_barrier(p.grid_bar, bar_base + (unsigned long long)gridDim.x, abortp)) fail(abortp, p.err_flag, 25);
    __syncthreads();
    barriers_done = 1;
  }
  uint32_t x_phase = 0, mma_phase = 0;  // parities of bar_x / bar_mma for this CTA's next active layer
  for (int l = 0; l < p.n_layers; ++l) {
    const ChainLayerParams& L = p.layer[l];
    const bool active = cta < L.n_tiles * L.splits;
    const int tile = active ? cta / L.splits : 0, slice = active ? cta % L.splits : 0;
    // the channel this thread requantises (its accumulator lane, or its share of the cluster's sum): the parameter
    // loads are in flight while the MMAs run
    const int per = clustered ? 128 / p.cluster : 128;  // channels of the tile this CTA finishes
    const int c_in_tile = clustered ? slice * per + (int)threadIdx.x % per : (int)threadIdx.x;
    const int ch = tile * 128 + c_in_tile;
    Requant rq;
    if (warp < 4 && active) rq.load(L, min(ch, L.N - 1));
    // the last layer may also write the DequantizeLinear that follows it: (q - zp) * scale as f32 lanes
    const bool tail = l + 1 == p.n_layers && p.tail_out != nullptr;
    auto store_out = [&](int row, uint8_t q) {
      L.out[(size_t)row * L.N + ch] = q;
      if (tail) p.tail_out[(size_t)row * L.N + ch] = __fmul_rn(__fsub_rn(p.tail_signed ? (float)(int)(int8_t)q : (float)q, p.tail_zp), p.tail_scale);
    };
    if (warp == 4) {
      // ---------------- loads and MMA issue ----------------
      if (active && !*abortp) {
        if (lane == 0) {
          // the rows were written by other CTAs through the generic proxy before the grid barrier
          asm volatile("fence.proxy.async;" ::: "memory");
          const uint32_t bar = smem_u32(&bar_x);
          mbar_expect_tx(bar, (uint32_t)L.kb * CHAIN_X_TILE);
          for (int i = 0; i < L.kb; ++i) tma_load_2d(base + p.x_off + (uint32_t)i * CHAIN_X_TILE, &L.tmX, bar, (slice * L.kb + i) * 128, 0);
        }
        __syncwarp();
        bool got = mbar_wait(smem_u32(&bar_w[l]), 0u, abortp);
        got = mbar_wait(smem_u32(&bar_x), x_phase, abortp) && got;
        x_phase ^= 1u;
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) fail(abortp, p.err_flag, 21);
        } else {
          tc_fence_after();
          if (lane == 0) {
            const uint64_t desc_rest = make_smem_desc(0, 128);
            const uint32_t desc_hi = (uint32_t)(desc_rest >> 32), desc_lo = (uint32_t)desc_rest;
            const uint32_t w16 = (base + L.w_off) >> 4, x16 = (base + p.x_off) >> 4;
            for (int i = 0; i < L.kb; ++i)
              tc_mma_block<KIND_I8, false>(tmem_base, desc_lo | ((w16 + (uint32_t)i * (CHAIN_W_TILE >> 4)) & 0x3fffu),
                                           desc_lo | ((x16 + (uint32_t)i * (CHAIN_X_TILE >> 4)) & 0x3fffu), desc_hi, L.idesc, i > 0 ? 1u : 0u, 4u);
            tc_commit<false>(smem_u32(&bar_mma));
          }
          __syncwarp();
          got = mbar_wait(smem_u32(&bar_mma), mma_phase, abortp);
          if (!__all_sync(0xffffffffu, got) && lane == 0) fail(abortp, p.err_flag, 22);
        }
        mma_phase ^= 1u;
      }
      // this layer's weight region is free now: start the loads of the layers that take it over
      if (lane == 0 && !*abortp)
        for (int l2 = l + 1; l2 < p.n_layers; ++l2)
          if (p.layer[l2].w_after == l) issue_weights(l2);
      __syncwarp();
    } else if (active) {
      // ---------------- accumulator lanes: channel = tile * 128 + 32 * warp + lane ----------------
      const bool got = mbar_wait(smem_u32(&bar_mma), mma_phase, abortp);
      mma_phase ^= 1u;
      const bool ok = __all_sync(0xffffffffu, got) && !*abortp;
      if (!ok && lane == 0) fail(abortp, p.err_flag, 23);
      const int cl = warp * 32 + lane;  // channel within the tile
      uint32_t v0[32], v1[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v0[j] = 0u, v1[j] = 0u;
      if (ok) {
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
        tmem_ld32_nowait(taddr, v0);
        tmem_ld32_nowait(taddr + 32u, v1);
        tmem_ld_wait_for(v0);
        tmem_ld_wait_for(v1);
        tc_fence_before();
      }
      if (clustered) {
        // partial sums into this CTA's shared memory, [row / 4][channel][row % 4]: the activation blocks, which the
        // MMAs have consumed, make room
#pragma unroll
        for (int g = 0; g < 8; ++g) dump[g * 128 + cl] = make_int4((int)v0[4 * g], (int)v0[4 * g + 1], (int)v0[4 * g + 2], (int)v0[4 * g + 3]);
#pragma unroll
        for (int g = 0; g < 8; ++g) dump[(8 + g) * 128 + cl] = make_int4((int)v1[4 * g], (int)v1[4 * g + 1], (int)v1[4 * g + 2], (int)v1[4 * g + 3]);
      } else {
        bool finish = ok;  // this CTA requantises the channel tile
        if (L.splits > 1) {
          // partial sums of this K slice: [tile][slice][row / 4][channel][row % 4], so that a warp's 16-byte stores
          // (and the last unit's loads) cover 512 contiguous bytes
          int4* ws_tile = reinterpret_cast<int4*>(L.ws) + (size_t)tile * L.splits * 16 * 128;
          int4* ws_mine = ws_tile + (size_t)slice * 16 * 128 + cl;
          if (ok) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (4 * g < p.rows) __stcg(ws_mine + g * 128, make_int4((int)v0[4 * g], (int)v0[4 * g + 1], (int)v0[4 * g + 2], (int)v0[4 * g + 3]));
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (32 + 4 * g < p.rows) __stcg(ws_mine + (8 + g) * 128, make_int4((int)v1[4 * g], (int)v1[4 * g + 1], (int)v1[4 * g + 2], (int)v1[4 * g + 3]));
          }
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 0) {
            unsigned int last = 0;
            if (ok) {
              const unsigned int old = atomicAdd(L.tile_count + tile, 1u);
              last = old == (unsigned int)(L.splits - 1) ? 1u : 0u;
              if (last) atomicExch(L.tile_count + tile, 0u);
            }
            last_slot = last;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          finish = last_slot != 0;
          if (finish) {
            __threadfence();
            for (int s2 = 0; s2 < L.splits; ++s2) {
              if (s2 == slice) continue;
              const int4* other = ws_tile + (size_t)s2 * 16 * 128 + cl;
#pragma unroll
              for (int g = 0; g < 8; ++g)
                if (4 * g < p.rows) {
                  const int4 t = __ldcg(other + g * 128);
                  v0[4 * g] += (uint32_t)t.x, v0[4 * g + 1] += (uint32_t)t.y, v0[4 * g + 2] += (uint32_t)t.z, v0[4 * g + 3] += (uint32_t)t.w;
                }
#pragma unroll
              for (int g = 0; g < 8; ++g)
                if (32 + 4 * g < p.rows) {
                  const int4 t = __ldcg(other + (8 + g) * 128);
                  v1[4 * g] += (uint32_t)t.x, v1[4 * g + 1] += (uint32_t)t.y, v1[4 * g + 2] += (uint32_t)t.z, v1[4 * g + 3] += (uint32_t)t.w;
                }
            }
          }
        }
        if (finish && ch < L.N) {
          uint8_t q0[32], q1[32];
          bool big = false;
#pragma unroll
          for (int r = 0; r < 32; ++r) q0[r] = rq.fast(v0[r], big), q1[r] = rq.fast(v1[r], big);
          if (big) {
#pragma unroll
            for (int r = 0; r < 32; ++r) q0[r] = rq.exact(v0[r]), q1[r] = rq.exact(v1[r]);
          }
#pragma unroll
          for (int r = 0; r < 32; ++r)
            if (r < p.rows) store_out(r, q0[r]);
#pragma unroll
          for (int r = 0; r < 32; ++r)
            if (32 + r < p.rows) store_out(32 + r, q1[r]);
        }
      }
    }
    if (clustered && cta < cluster_units(L, p.cluster)) {
      // ---------------- the K slices of a channel tile are the CTAs of one cluster: sum through distributed shared memory ----
      // CTA `slice` of the cluster owns channels [32 * slice', ...) in steps of the cluster size; every thread of the
      // cluster takes part in both barriers whatever happened before, so nobody waits for a CTA that gave up
      cluster_sync_all();
      if (warp < 4) {
        const int rg = (int)threadIdx.x / per;     // row group: 128 / per groups of 64 * per / 128 rows
        const int rows_per = 64 * per / 128;       // 16 for a cluster of 4
        const uint32_t dump_addr = base + p.x_off;
        uint32_t acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
#pragma unroll
        for (int src = 0; src < 8; ++src) {
          if (src >= p.cluster) break;
          const uint32_t remote = mapa(dump_addr, (uint32_t)src);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            if (4 * g < rows_per) {
              const int r4 = rg * (rows_per / 4) + g;
              const int4 t = ld_dsmem_v4(remote + (uint32_t)(r4 * 128 + c_in_tile) * 16u);
              acc[4 * g] += (uint32_t)t.x, acc[4 * g + 1] += (uint32_t)t.y, acc[4 * g + 2] += (uint32_t)t.z, acc[4 * g + 3] += (uint32_t)t.w;
            }
        }
        if (ch < L.N && !*abortp) {
          uint8_t q[32];
          bool big = false;
#pragma unroll
          for (int r = 0; r < 32; ++r) q[r] = rq.fast(acc[r], big);
          if (big) {
#pragma unroll
            for (int r = 0; r < 32; ++r) q[r] = rq.exact(acc[r]);
          }
#pragma unroll
          for (int r = 0; r < 32; ++r) {
            const int row = rg * rows_per + r;
            if (r < rows_per && row < p.rows) store_out(row, q[r]);
          }
        }
      }
      // Peers may still be reading this CTA's partial sums.  Between layers the grid barrier below covers that (a
      // peer arrives there only after its reads, and nothing overwrites the partial sums before it); the last
      // layer has no grid barrier, and the CTA's shared memory must outlive the peers' reads.
      if (l + 1 == p.n_layers) cluster_sync_all();
    }
    if (l + 1 < p.n_layers) {
      // every CTA's rows of this layer are visible (also to the TMA unit) before anybody loads the next layer's
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");
      tc_fence_before();
      __syncthreads();
      if (threadIdx.x == 0 && !*abortp) {
        if (!grid_barrier(p.grid_bar, bar_base + (unsigned long long)(barriers_done + l + 1) * gridDim.x, abortp)) fail(abortp, p.err_flag, 24);
      }
      __syncthreads();
      tc_fence_after();
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
  if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(CHAIN_ROWS) : "memory");
}

// [N][K] 8-bit weights -> [channel tile][K block][128 channels][128 bytes of K], channels beyond N zero: what one
// TMA load of the chain kernel fetches is then 16 KB contiguous instead of 128 pieces a whole weight row apart
// (cold from HBM, the strided form ran at a fraction of the copy bandwidth).
__global__ void chain_repack_kernel(const uint4* __restrict__ w, uint4* __restrict__ out, int N, int K, int64_t total16) {
  const int kblocks = K / 128;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total16; o += (int64_t)gridDim.x * blockDim.x) {
    const int piece = (int)(o & 7), c = (int)((o >> 3) & 127);
    const int64_t blk = o >> 10;
    const int kb = (int)(blk % kblocks), tile = (int)(blk / kblocks);
    const int ch = tile * 128 + c;
    out[o] = ch < N ? w[((int64_t)ch * K + kb * 128) / 16 + piece] : make_uint4(0u, 0u, 0u, 0u);
  }
}

void chain_repack(const void* w, void* out, int N, int K, cudaStream_t s) {
  const int64_t total16 = (int64_t)((N + 127) / 128) * 128 * K / 16;
  const int64_t blocks = std::min<int64_t>((total16 + 255) / 256, 148 * 16);
  chain_repack_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint4*)w, (uint4*)out, N, K, total16);
}

namespace {

void ensure_chain_smem(size_t smem, int device) {
  static std::mutex mu;
  static size_t have[kMaxDevices] = {};
  const int d = (device >= 0 && device < kMaxDevices) ? device : 0;
  std::lock_guard<std::mutex> lock(mu);
  if (smem > have[d]) {
    OXB_CUDA(cudaFuncSetAttribute(umma_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    have[d] = smem;
  }
}

}  // namespace

// A cooperative launch: the grid-wide barrier needs every CTA resident at once, which the driver then guarantees
// (or refuses the launch).
static cudaError_t launch_chain_raw(const ChainParams& p, int grid, size_t smem, int device, int cluster, cudaStream_t s) {
  ensure_chain_smem(smem, device);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(CHAIN_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  int n_attr = 1;
  if (cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    n_attr = 2;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, umma_chain_kernel, p);
}

bool launch_chain(const ChainParams& p, int grid, size_t smem, int device, int cluster, cudaStream_t s) {
  if (launch_chain_raw(p, grid, smem, device, cluster, s) == cudaSuccess) return true;
  (void)cudaGetLastError();  // a refused launch (co-residency not available right now) ran nothing
  return false;
}

bool try_launch_chain(const ChainParams& p, int grid, size_t smem, int device, int cluster) {
  if (launch_chain_raw(p, grid, smem, device, cluster, nullptr) != cudaSuccess || cudaStreamSynchronize(nullptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return true;
}

int chain_max_resident(size_t smem, int device, int cluster) {
  ensure_chain_smem(smem, device);
  if (cluster > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(CHAIN_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, umma_chain_kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      return 0;
    }
    return n * cluster;
  }
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, umma_chain_kernel, CHAIN_THREADS, smem) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return per_sm * sms;
}

}  // namespace umma
}  // namespace k
}  // namespace oxb
