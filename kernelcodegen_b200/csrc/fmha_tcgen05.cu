// Fused multi-head attention forward (placeholder until the tcgen05 kernel lands).
#include "common.cuh"

extern "C" int kcg_fmha_fwd(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                            float softmax_scale, int causal, const void* Q, const int64_t q_strides[3],
                            const void* K, const int64_t k_strides[3], const void* V,
                            const int64_t v_strides[3], void* O, const int64_t o_strides[3], void* stream) {
  using namespace kcg;
  clear_error();
  return fail(KCG_ERR_UNSUPPORTED, "fmha: kernel not built");
}
