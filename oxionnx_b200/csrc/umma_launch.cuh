// Launch templates of the tcgen05 kernel; included by the one translation unit per kind.
#pragma once

#include <mutex>

#include "umma_kernel.cuh"

namespace oxb {
namespace k {
namespace umma {

// The opt-in for more than 48 KB of dynamic shared memory is a per-device property of a kernel: it is recorded
// per (instantiation, device) and set again whenever a plan needs more, under a lock, with that device current.
template <int BN, int KIND, bool PAIR>
void ensure_smem_attr(size_t smem, int device) {
  static std::mutex mu;
  static size_t have[kMaxDevices] = {};
  const int d = (device >= 0 && device < kMaxDevices) ? device : 0;
  std::lock_guard<std::mutex> lock(mu);
  if (smem > have[d]) {
    OXB_CUDA(cudaFuncSetAttribute(umma_conv_kernel<BN, KIND, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    have[d] = smem;
  }
}

template <int BN, int KIND, bool PAIR>
void launch_one(const KParams& kp, int grid, size_t smem, int device, cudaStream_t s) {
  ensure_smem_attr<BN, KIND, PAIR>(smem, device);
  // Programmatic dependent launch: this grid may be scheduled while its predecessor in the stream drains, so
  // that its prologue (barrier setup, TMEM allocation) overlaps the predecessor's tail; it touches no global
  // memory before griddepcontrol.wait, which returns only once the predecessor has completed and flushed.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(64 + 32 * epi_warps(KIND));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  int n_attr = 1;
  if (PAIR) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    n_attr = 2;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  OXB_CUDA(cudaLaunchKernelEx(&cfg, umma_conv_kernel<BN, KIND, PAIR>, kp));
}

template <int BN, int KIND, bool PAIR>
int max_clusters_one(size_t smem, int device) {
  ensure_smem_attr<BN, KIND, PAIR>(smem, device);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148);
  cfg.blockDim = dim3(64 + 32 * epi_warps(KIND));
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, umma_conv_kernel<BN, KIND, PAIR>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

template <int KIND>
void launch_any(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s) {
  if (pair) {
    if (bn != 256) OXB_FAIL("umma_launch: a CTA pair needs the 256-wide tile, not %d", bn);
    launch_one<256, KIND, true>(kp, grid, smem, device, s);
    return;
  }
  switch (bn) {
    case 32: launch_one<32, KIND, false>(kp, grid, smem, device, s); break;
    case 64: launch_one<64, KIND, false>(kp, grid, smem, device, s); break;
    case 128: launch_one<128, KIND, false>(kp, grid, smem, device, s); break;
    case 256: launch_one<256, KIND, false>(kp, grid, smem, device, s); break;
    default: OXB_FAIL("umma_launch: unsupported tile width %d", bn);
  }
}

template <int KIND>
int max_pairs_any(size_t smem, int device) {
  return max_clusters_one<256, KIND, true>(smem, device);
}

}  // namespace umma
}  // namespace k
}  // namespace oxb
