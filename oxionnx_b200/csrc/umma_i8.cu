// Instantiations of the tcgen05 implicit-GEMM kernel for kind::i8 (all tile widths, lone CTAs and CTA pairs).
#include "umma_launch.cuh"

namespace oxb {
namespace k {
namespace umma {

void launch_kind_i8(const KParams& kp, int bn, bool pair, int grid, size_t smem, int device, cudaStream_t s) {
  launch_any<KIND_I8>(kp, bn, pair, grid, smem, device, s);
}
int max_pairs_kind_i8(size_t smem, int device) { return max_pairs_any<KIND_I8>(smem, device); }

}  // namespace umma
}  // namespace k
}  // namespace oxb
