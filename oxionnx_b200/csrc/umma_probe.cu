// Issue-rate probe of the tensor pipe: every SM issues a long run of 128 x 256 x (32 bytes of K) tcgen05.mma
// instructions on shared memory that is never refilled (all zeros), so nothing but the tensor pipe itself
// bounds the time.  The result is the peak a contraction kernel of that kind could reach on this device at the
// clocks it ran at; the roofline fractions of the benchmark quote it next to the cuBLAS-derived figures.
#include <cuda.h>

#include "umma_kernel.cuh"

namespace oxb {
namespace k {
namespace {

using namespace umma;

template <int KIND>
__global__ void __launch_bounds__(128, 1) probe_kernel(int groups, uint32_t idesc, int* err) {
  extern __shared__ uint8_t raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  uint32_t* words = reinterpret_cast<uint32_t*>(raw + (base - smem_u32(raw)));
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) words[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (warp == 0) {
    bool ok = true;
    if (lane == 0) {
      const uint64_t desc = make_smem_desc(0, 128);
      const uint32_t desc_hi = (uint32_t)(desc >> 32), desc_lo = (uint32_t)desc;
      const uint32_t a16 = base >> 4, b16 = (base + 16384u) >> 4;
      // four instructions (one 128-byte K block) per group, two accumulators in turn
      for (int g = 0; g < groups; ++g)
        tc_mma_block<KIND, false>(tm + (uint32_t)(g & 1) * 256u, desc_lo | (a16 & 0x3fffu), desc_lo | (b16 & 0x3fffu), desc_hi, idesc, g >= 2 ? 1u : 0u, 4u);
      tc_commit<false>(smem_u32(&bar));
      const long long start = clock64();
      while (!mbar_try_wait(smem_u32(&bar), 0)) {
        if (clock64() - start > WAIT_CYCLES) {
          ok = false;
          break;
        }
      }
      if (!ok) atomicExch(err, 9);
    }
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
}

uint32_t probe_idesc(int kind) {
  uint32_t d = 0;
  if (kind == KIND_I8) d |= (2u << 4) | (1u << 10);                          // s32 accumulator, A u8, B s8
  else if (kind == KIND_TF32) d |= (1u << 4) | (2u << 7) | (2u << 10);      // f32 accumulator, tf32 operands
  else d |= (1u << 4) | ((kind == KIND_BF16 ? 1u : 0u) << 7) | ((kind == KIND_BF16 ? 1u : 0u) << 10);
  d |= (uint32_t)(256 >> 3) << 17;
  d |= (uint32_t)(BLOCK_M >> 4) << 24;
  return d;
}

template <int KIND>
float run_probe(int grid, int groups, uint32_t idesc, int* err, cudaStream_t s) {
  const size_t smem = 49 * 1024 + 1024;
  OXB_CUDA(cudaFuncSetAttribute(probe_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaEvent_t e0, e1;
  OXB_CUDA(cudaEventCreate(&e0));
  OXB_CUDA(cudaEventCreate(&e1));
  float best = 1e30f;
  for (int rep = 0; rep < 4; ++rep) {
    OXB_CUDA(cudaEventRecord(e0, s));
    probe_kernel<KIND><<<grid, 128, smem, s>>>(groups, idesc, err);
    OXB_CUDA(cudaEventRecord(e1, s));
    OXB_CUDA(cudaStreamSynchronize(s));
    float ms = 0.f;
    OXB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (rep > 0 && ms < best) best = ms;  // the first launch pays the module load
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  OXB_CUDA(cudaGetLastError());
  return best;
}

}  // namespace

// Operations (2 per multiply-add) per second of the tensor pipe for `kind`, all SMs issuing; fails when a wait ran out.
double umma_probe_peak(int kind, int* err_flag, cudaStream_t s) {
  int dev = 0, sms = 148;
  OXB_CUDA(cudaGetDevice(&dev));
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int groups = 8192;  // 32768 instructions of 128 tensor-pipe cycles each: about 2 ms
  const uint32_t idesc = probe_idesc(kind);
  float ms;
  if (kind == KIND_I8) ms = run_probe<KIND_I8>(sms, groups, idesc, err_flag, s);
  else if (kind == KIND_TF32) ms = run_probe<KIND_TF32>(sms, groups, idesc, err_flag, s);
  else ms = run_probe<KIND_F16>(sms, groups, idesc, err_flag, s);
  const double k_per_instr = 32.0 / umma_elem_bytes(kind);
  const double ops = 2.0 * (double)sms * groups * 4.0 * BLOCK_M * 256.0 * k_per_instr;
  return ops / ((double)ms * 1e-3);
}

}  // namespace k
}  // namespace oxb
