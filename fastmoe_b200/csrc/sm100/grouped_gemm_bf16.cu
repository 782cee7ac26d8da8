// bf16 instantiations of the grouped GEMM kernel.
#include "grouped_gemm_kernel.cuh"

namespace fmoe {
namespace gg {
cudaError_t launch_bf16(int mode, const CUtensorMap& ta, const CUtensorMap& tb,
                        const KernelParams& kp, int grid, cudaStream_t stream) {
  return launch_for_type<__nv_bfloat16>(mode, ta, tb, kp, grid, stream);
}
}  // namespace gg
}  // namespace fmoe
