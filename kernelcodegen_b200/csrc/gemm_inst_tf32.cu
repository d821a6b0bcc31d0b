// Instantiation unit of the tensor-core GEMM kernels (gemm_kernels.cuh): tf32 operands (both K-major: the fp32 path lays them out that way), fp32 output.
#include "gemm_kernels.cuh"

namespace kcg {

int gemm_launch_tf32(KCG_GEMM_LAUNCH_ARGS) {
  (void)trans_a; (void)trans_b;
  return launch_variant<Kind::TF32, 4, false, false, float>(tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace kcg
