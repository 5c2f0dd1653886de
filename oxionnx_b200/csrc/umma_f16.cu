// Instantiations of the tcgen05 implicit-GEMM kernel for kind::f16 (all tile widths, lone CTAs and CTA pairs).
#include "umma_launch.cuh"

namespace oxb {
namespace k {
namespace umma {

void launch_kind_f16(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s) {
  launch_any<KIND_F16>(kp, bn, pair, grid, smem, device, s);
}
int max_pairs_kind_f16(size_t smem, int device) { return max_pairs_any<KIND_F16>(smem, device); }

}  // namespace umma
}  // namespace k
}  // namespace oxb
