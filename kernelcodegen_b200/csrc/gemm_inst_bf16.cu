// Instantiation unit of the tensor-core GEMM kernels (gemm_kernels.cuh): bf16 operands, bf16 output.
#include "gemm_kernels.cuh"

namespace kcg {

int gemm_launch_f16kind_bf16(KCG_GEMM_LAUNCH_ARGS) {
  return launch_layout<Kind::F16, 2, __nv_bfloat16>(trans_a, trans_b, tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace kcg
