// Instantiation unit of the tensor-core GEMM kernels (gemm_kernels.cuh): bf16 or fp16 operands (the instruction descriptor says which), fp32 output.
#include "gemm_kernels.cuh"

namespace kcg {

int gemm_launch_f16kind_f32(KCG_GEMM_LAUNCH_ARGS) {
  return launch_layout<Kind::F16, 2, float>(trans_a, trans_b, tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace kcg
