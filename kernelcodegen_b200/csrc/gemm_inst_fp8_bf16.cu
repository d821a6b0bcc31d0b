// Instantiation unit of the tensor-core GEMM kernels (gemm_kernels.cuh): e4m3 operands, bf16 output.
#include "gemm_kernels.cuh"

namespace kcg {

int gemm_launch_f8_bf16(KCG_GEMM_LAUNCH_ARGS) {
  return launch_layout<Kind::F8F6F4, 1, __nv_bfloat16>(trans_a, trans_b, tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace kcg
