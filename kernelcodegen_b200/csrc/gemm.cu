// kcg_gemm: argument checking and the choice between the tensor-core kernel
// (gemm_tcgen05.cu) and the fp32 CUDA-core kernel (sgemm.cu).
#include "common.cuh"

namespace kcg {
int sgemm_f32(int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a, int trans_b, const float* A,
              int64_t lda, int64_t stride_a, const float* B, int64_t ldb, int64_t stride_b, float* C,
              int64_t ldc, int64_t stride_c, const float* scale_a, const float* scale_b, const float* bias, int act,
              cudaStream_t stream);
int gemm_tcgen05(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a,
                 int trans_b, const void* A, int64_t lda, int64_t stride_a, const void* B, int64_t ldb,
                 int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, const float* scale_a,
                 const float* scale_b, const void* bias, int act, cudaStream_t stream, void* const* extra_c = nullptr,
                 int n_extra = 0, void* mc_c = nullptr);
int gemm_f32_tensor(int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a, int trans_b, const float* A,
                    int64_t lda, int64_t stride_a, const float* B, int64_t ldb, int64_t stride_b, float* C,
                    int64_t ldc, int64_t stride_c, const float* scale_a, const float* scale_b, const float* bias,
                    int act, cudaStream_t stream);
namespace {
thread_local int g_fp32_mode = -1;  // per calling thread; -1: by size; 0: CUDA-core kernel; 1: tensor cores (three tf32 products)
}
}  // namespace kcg

extern "C" void kcg_gemm_set_fp32_mode(int mode) { kcg::g_fp32_mode = mode; }

extern "C" int kcg_gemm(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int64_t batch,
                        int trans_a, int trans_b, const void* A, int64_t lda, int64_t stride_a,
                        const void* B, int64_t ldb, int64_t stride_b, void* C, int64_t ldc,
                        int64_t stride_c, const float* scale_a, const float* scale_b, void* stream) {
  return kcg_gemm_fused(dtype_in, dtype_out, M, N, K, batch, trans_a, trans_b, A, lda, stride_a, B, ldb, stride_b, C,
                        ldc, stride_c, scale_a, scale_b, nullptr, 0, stream);
}

extern "C" int kcg_gemm_fused(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int64_t batch,
                              int trans_a, int trans_b, const void* A, int64_t lda, int64_t stride_a,
                              const void* B, int64_t ldb, int64_t stride_b, void* C, int64_t ldc,
                              int64_t stride_c, const float* scale_a, const float* scale_b,
                              const void* bias, int activation, void* stream) {
  using namespace kcg;
  clear_error();
  if (activation < 0 || activation > 2) return fail(KCG_ERR_INVALID_ARG, "gemm: activation %d (0 none, 1 Relu, 2 Gelu)", activation);
  if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(KCG_ERR_INVALID_ARG, "gemm: negative extent");
  if (M == 0 || N == 0 || batch == 0) return KCG_OK;
  if (K == 0) return fail(KCG_ERR_INVALID_ARG, "gemm: K must be positive");
  if (!A || !B || !C) return fail(KCG_ERR_INVALID_ARG, "gemm: null pointer");
  const int64_t a_cols = trans_a ? M : K, b_cols = trans_b ? K : N;
  if (lda < a_cols || ldb < b_cols || ldc < N)
    return fail(KCG_ERR_INVALID_ARG,
                "gemm: leading dimension shorter than a row (lda=%lld need %lld, ldb=%lld need %lld, ldc=%lld need %lld)",
                static_cast<long long>(lda), static_cast<long long>(a_cols), static_cast<long long>(ldb),
                static_cast<long long>(b_cols), static_cast<long long>(ldc), static_cast<long long>(N));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype_in == KCG_F32) {
    if (dtype_out != KCG_F32) return fail(KCG_ERR_UNSUPPORTED, "gemm: float32 inputs produce float32");
    // Large enough products go to the tensor cores as three tf32 products of split operands
    // (results within ~1e-6 of fp64); small ones, where the two split passes would dominate,
    // and anything the split path declines stay on the CUDA-core kernel.
    const bool big = static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K) >= 256.0 * 256.0 * 256.0;
    if (g_fp32_mode == 1 || (g_fp32_mode == -1 && big)) {
      const int rc = gemm_f32_tensor(M, N, K, batch, trans_a, trans_b, static_cast<const float*>(A), lda, stride_a,
                                     static_cast<const float*>(B), ldb, stride_b, static_cast<float*>(C), ldc, stride_c,
                                     scale_a, scale_b, static_cast<const float*>(bias), activation, s);
      if (rc != KCG_ERR_UNSUPPORTED || kcg_last_error()[0] != 0) return rc;
    }
    return sgemm_f32(M, N, K, batch, trans_a, trans_b, static_cast<const float*>(A), lda, stride_a,
                     static_cast<const float*>(B), ldb, stride_b, static_cast<float*>(C), ldc, stride_c,
                     scale_a, scale_b, static_cast<const float*>(bias), activation, s);
  }
  if (dtype_in == KCG_BF16 || dtype_in == KCG_F16 || dtype_in == KCG_F8E4M3)
    return gemm_tcgen05(dtype_in, dtype_out, M, N, K, batch, trans_a, trans_b, A, lda, stride_a, B, ldb,
                        stride_b, C, ldc, stride_c, scale_a, scale_b, bias, activation, s);
  return fail(KCG_ERR_UNSUPPORTED, "gemm: input dtype %d has no kernel", dtype_in);
}

// GEMM whose epilogue also performs the all-gather of C: every output tile is stored into
// this rank's row block of each rank's gathered matrix (gathered[r], r < world), the local one
// included, with plain stores — to peer GPUs through their mapped memory.
extern "C" int kcg_gemm_allgather(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int trans_a,
                                  int trans_b, const void* A, int64_t lda, const void* B, int64_t ldb,
                                  void* const* gathered, int world, int rank, int64_t row_offset, int64_t ldc,
                                  const float* scale_a, const float* scale_b, const void* bias, int activation,
                                  void* stream) {
  using namespace kcg;
  clear_error();
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(KCG_ERR_INVALID_ARG, "gemm_allgather: world %d (1..8), rank %d", world, rank);
  if (!gathered) return fail(KCG_ERR_INVALID_ARG, "gemm_allgather: null pointer");
  if (row_offset < 0 || ldc < N) return fail(KCG_ERR_INVALID_ARG, "gemm_allgather: bad row offset or ldc");
  if (activation < 0 || activation > 2) return fail(KCG_ERR_INVALID_ARG, "gemm: activation %d (0 none, 1 Relu, 2 Gelu)", activation);
  if (M < 0 || N < 0 || K < 0) return fail(KCG_ERR_INVALID_ARG, "gemm: negative extent");
  if (M == 0 || N == 0) return KCG_OK;
  if (K == 0) return fail(KCG_ERR_INVALID_ARG, "gemm: K must be positive");
  if (!A || !B) return fail(KCG_ERR_INVALID_ARG, "gemm: null pointer");
  if (dtype_in != KCG_BF16 && dtype_in != KCG_F16 && dtype_in != KCG_F8E4M3)
    return fail(KCG_ERR_UNSUPPORTED, "gemm_allgather: tensor-core input dtypes only (bfloat16, float16, float8_e4m3)");
  const int64_t a_cols = trans_a ? M : K, b_cols = trans_b ? K : N;
  if (lda < a_cols || ldb < b_cols) return fail(KCG_ERR_INVALID_ARG, "gemm: leading dimension shorter than a row");
  const size_t out_es = kcg_dtype_size(dtype_out);
  void* mine = nullptr;
  void* others[8];
  int n_others = 0;
  for (int r = 0; r < world; ++r) {
    if (!gathered[r]) return fail(KCG_ERR_INVALID_ARG, "gemm_allgather: gathered[%d] is null", r);
    void* blk = static_cast<char*>(gathered[r]) + static_cast<size_t>(row_offset) * ldc * out_es;
    if (r == rank) mine = blk; else others[n_others++] = blk;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return gemm_tcgen05(dtype_in, dtype_out, M, N, K, 1, trans_a, trans_b, A, lda, 0, B, ldb, 0, mine, ldc, 0, scale_a,
                      scale_b, bias, activation, s, others, n_others);
}

// The same with the gather done by NVSwitch: every tile is stored once, to the multicast address
// of its place in the gathered matrix, and arrives in every rank's buffer (this rank's included).
extern "C" int kcg_gemm_allgather_multicast(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int trans_a,
                                            int trans_b, const void* A, int64_t lda, const void* B, int64_t ldb,
                                            void* gathered_local, void* gathered_multicast, int64_t row_offset,
                                            int64_t ldc, const float* scale_a, const float* scale_b, const void* bias,
                                            int activation, void* stream) {
  using namespace kcg;
  clear_error();
  if (!gathered_local || !gathered_multicast) return fail(KCG_ERR_INVALID_ARG, "gemm_allgather_multicast: null pointer");
  if (row_offset < 0 || ldc < N) return fail(KCG_ERR_INVALID_ARG, "gemm_allgather_multicast: bad row offset or ldc");
  if (activation < 0 || activation > 2) return fail(KCG_ERR_INVALID_ARG, "gemm: activation %d (0 none, 1 Relu, 2 Gelu)", activation);
  if (M < 0 || N < 0 || K < 0) return fail(KCG_ERR_INVALID_ARG, "gemm: negative extent");
  if (M == 0 || N == 0) return KCG_OK;
  if (K == 0) return fail(KCG_ERR_INVALID_ARG, "gemm: K must be positive");
  if (!A || !B) return fail(KCG_ERR_INVALID_ARG, "gemm: null pointer");
  if (dtype_in != KCG_BF16 && dtype_in != KCG_F16 && dtype_in != KCG_F8E4M3)
    return fail(KCG_ERR_UNSUPPORTED, "gemm_allgather_multicast: tensor-core input dtypes only (bfloat16, float16, float8_e4m3)");
  const int64_t a_cols = trans_a ? M : K, b_cols = trans_b ? K : N;
  if (lda < a_cols || ldb < b_cols) return fail(KCG_ERR_INVALID_ARG, "gemm: leading dimension shorter than a row");
  const size_t shift = static_cast<size_t>(row_offset) * ldc * kcg_dtype_size(dtype_out);
  return gemm_tcgen05(dtype_in, dtype_out, M, N, K, 1, trans_a, trans_b, A, lda, 0, B, ldb, 0,
                      static_cast<char*>(gathered_local) + shift, ldc, 0, scale_a, scale_b, bias, activation,
                      static_cast<cudaStream_t>(stream), nullptr, 0, static_cast<char*>(gathered_multicast) + shift);
}
