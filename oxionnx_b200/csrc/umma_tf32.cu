// Instantiations of the tcgen05 implicit-GEMM kernel for kind::tf32 (all tile widths, lone CTAs and CTA pairs).
#include "umma_launch.cuh"

namespace oxb {
namespace k {
namespace umma {

void launch_kind_tf32(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s) {
  launch_any<KIND_TF32>(kp, bn, pair, grid, smem, device, s);
}
int max_pairs_kind_tf32(size_t smem, int device) { return max_pairs_any<KIND_TF32>(smem, device); }

}  // namespace umma
}  // namespace k
}  // namespace oxb
