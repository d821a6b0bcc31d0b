// Instantiation unit of the tensor-core GEMM kernels (gemm_kernels.cuh): fp16 operands, fp16 output.
#include "gemm_kernels.cuh"

namespace kcg {

int gemm_launch_f16kind_f16(KCG_GEMM_LAUNCH_ARGS) {
  return launch_layout<Kind::F16, 2, __half>(trans_a, trans_b, tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace kcg
