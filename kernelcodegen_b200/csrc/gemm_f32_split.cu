// fp32 GEMM on the tensor cores by operand splitting.
//
// tcgen05 has no fp32 x fp32 MMA; kind::tf32 reads fp32 words but keeps 10 mantissa bits, which
// alone cannot meet a 1e-5 tolerance.  Writing each operand as hi + lo with hi = tf32(x) and
// lo = tf32(x - hi) (x - hi is exact in fp32) gives
//     a b  =  a_hi b_hi + a_lo b_hi + a_hi b_lo  +  O(2^-21 |a b|),
// and the three products are exact in the fp32 accumulator, so one tf32 GEMM over the
// concatenated operands  A' = [A_hi | A_lo | A_hi]  (M x 3K)  and  B' = [B_hi | B_hi | B_lo]
// (N x 3K, K-major) yields fp32-grade results (relative error ~1e-6 at K = 1024) at a third
// of the tf32 rate — several times the CUDA-core kernel.
//
// The tensor core's accumulator does not round to nearest: measured, the error of a long tf32
// accumulation grows linearly with K (about 1e-8 K relative), which would break 1e-5 beyond
// K ~ 900.  So K is cut into chunks of 256: each chunk is one entry of a batched GEMM writing an
// fp32 partial product, and a second kernel adds the partials in ordinary fp32 arithmetic and
// applies the epilogue (scales, bias, activation).  The split operands and the partials live in
// a per-device scratch buffer (slot 1 of the library's cached allocations).
#include <algorithm>

#include "common.cuh"

namespace kcg {
int gemm_tcgen05(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a,
                 int trans_b, const void* A, int64_t lda, int64_t stride_a, const void* B, int64_t ldb,
                 int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, const float* scale_a,
                 const float* scale_b, const void* bias, int act, cudaStream_t stream, void* const* extra_c,
                 int n_extra, void* mc_c = nullptr);
void* device_scratch(size_t bytes, int slot, cudaStream_t stream, int* why);  // runtime.cu

namespace {

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// hi / lo parts of x; an infinite or NaN x keeps its value in hi and gets lo = 0.
__device__ __forceinline__ void split(float x, float& hi, float& lo) {
  hi = tf32_round(x);
  const float d = x - hi;
  lo = (d == d && fabsf(hi) != INFINITY) ? tf32_round(d) : 0.f;
}

constexpr int64_t kChunkK = 256;   // original K per chunk (768 tf32 columns after splitting)

// Destination layout: [batch][chunk][row][3 * kc] with kc = min(kChunkK, Kp); a row holds the
// three kc-long thirds (hi, lo, hi) for kOrder 0 or (hi, hi, lo) for kOrder 1; columns past K
// are zero padding.
template <int kOrder>
__device__ __forceinline__ void store_split(float* dst, int64_t b, int64_t rows, int64_t r, int64_t k, int64_t kc,
                                            int64_t chunks, float x, bool valid) {
  float hi = 0.f, lo = 0.f;
  if (valid) split(x, hi, lo);
  const int64_t c = k / kc, kk = k % kc;
  float* drow = dst + ((b * chunks + c) * rows + r) * 3 * kc;
  drow[kk] = hi;
  drow[kc + kk] = kOrder == 0 ? lo : hi;
  drow[2 * kc + kk] = kOrder == 0 ? hi : lo;
}

// Source rows are contiguous along k: src(r, k) = src[r * ld + k].
template <int kOrder>
__global__ void __launch_bounds__(256)
split_k_contiguous(const float* __restrict__ src, int64_t rows, int64_t K, int64_t ld, int64_t src_batch,
                   float* __restrict__ dst, int64_t Kp, int64_t kc, int64_t chunks) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t k = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = blockIdx.y;
  if (k >= Kp) return;
  const float* s = src + blockIdx.z * src_batch + r * ld;
  store_split<kOrder>(dst, blockIdx.z, rows, r, k, kc, chunks, k < K ? s[k] : 0.f, k < K);
}

// Source is contiguous along the row index: src(r, k) = src[k * ld + r]; 32 x 32 tiles through
// shared memory so that both the read and the write are coalesced.
template <int kOrder>
__global__ void __launch_bounds__(256)
split_r_contiguous(const float* __restrict__ src, int64_t rows, int64_t K, int64_t ld, int64_t src_batch,
                   float* __restrict__ dst, int64_t Kp, int64_t kc, int64_t chunks) {
  __shared__ float tile[32][33];
  grid_launch_dependents();
  grid_dependency_wait();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * 32, k0 = static_cast<int64_t>(blockIdx.y) * 32;
  const float* s = src + blockIdx.z * src_batch;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t k = k0 + ty + 8 * i, r = r0 + tx;
    tile[ty + 8 * i][tx] = (k < K && r < rows) ? s[k * ld + r] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + ty + 8 * i, k = k0 + tx;
    if (r < rows && k < Kp) store_split<kOrder>(dst, blockIdx.z, rows, r, k, kc, chunks, tile[tx][ty + 8 * i], k < K);
  }
}

// C = epilogue(sum over chunks of the partial products), added in chunk order in fp32.
__global__ void __launch_bounds__(256)
reduce_partials(const float* __restrict__ part, int64_t chunks, int64_t M, int64_t N, float* __restrict__ C, int64_t ldc,
                int64_t stride_c, const float* __restrict__ scale_a, const float* __restrict__ scale_b,
                const float* __restrict__ bias, int act) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t n4 = (N + 3) / 4;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= M * n4) return;
  const int64_t m = t / n4, n0 = (t % n4) * 4;
  const int64_t b = blockIdx.y;
  float alpha = 1.f;
  if (scale_a) alpha *= *scale_a;
  if (scale_b) alpha *= *scale_b;
  const float* p = part + (b * chunks * M + m) * N + n0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const bool vec = (N % 4 == 0);
  for (int64_t c = 0; c < chunks; ++c, p += M * N) {
    if (vec) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(p));
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < N) acc[j] += p[j];
    }
  }
  float* crow = C + b * stride_c + m * ldc + n0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (n0 + j < N) crow[j] = gemm_epilogue_value<float>(acc[j], alpha, bias, n0 + j, act);
}

template <int kOrder>
int launch_split(const float* src, bool k_contiguous, int64_t rows, int64_t K, int64_t ld, int64_t src_batch,
                 int64_t batch, float* dst, int64_t Kp, int64_t kc, int64_t chunks, cudaStream_t stream) {
  if (rows > 65535ll * 32 || batch > 65535) return fail(KCG_ERR_UNSUPPORTED, "fp32 gemm (tensor path): extent too large");
  if (k_contiguous) {
    if (rows > 65535) return fail(KCG_ERR_UNSUPPORTED, "fp32 gemm (tensor path): more than 65535 rows");
    dim3 grid(static_cast<unsigned>((Kp + 255) / 256), static_cast<unsigned>(rows), static_cast<unsigned>(batch));
    launch_overlapped(split_k_contiguous<kOrder>, grid, dim3(256), 0, stream, src, rows, K, ld, src_batch, dst, Kp, kc, chunks);
  } else {
    const int64_t gy = (Kp + 31) / 32;
    if (gy > 65535) return fail(KCG_ERR_UNSUPPORTED, "fp32 gemm (tensor path): K too large");
    dim3 grid(static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
    launch_overlapped(split_r_contiguous<kOrder>, grid, dim3(256), 0, stream, src, rows, K, ld, src_batch, dst, Kp, kc, chunks);
  }
  return check_launch("split_tf32");
}

}  // namespace

// Returns KCG_ERR_UNSUPPORTED (without a message) when the problem should stay on the CUDA-core
// kernel: operands too large for the scratch buffer.
int gemm_f32_tensor(int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a, int trans_b, const float* A,
                    int64_t lda, int64_t stride_a, const float* B, int64_t ldb, int64_t stride_b, float* C,
                    int64_t ldc, int64_t stride_c, const float* scale_a, const float* scale_b, const float* bias,
                    int act, cudaStream_t stream) {
  // K padded to whole chunks (or to a multiple of 8 when one chunk covers it)
  const int64_t kc = K <= kChunkK ? (K + 7) / 8 * 8 : kChunkK;
  const int64_t chunks = (K + kc - 1) / kc, Kp = chunks * kc, kc3 = 3 * kc;
  const size_t op_floats = static_cast<size_t>(batch) * static_cast<size_t>(M + N) * 3 * Kp;
  // The partial products of all chunks are kept for a panel of columns at a time, so that they
  // never need more than about 1 GiB: C is produced panel by panel.
  int64_t panel = N;
  if (chunks > 1) {
    const int64_t cap_cols = (1ll << 28) / (batch * chunks * M);   // floats in 1 GiB / rows of partials
    if (cap_cols < N) panel = cap_cols / 256 * 256;
    if (panel < 256) return KCG_ERR_UNSUPPORTED;
  }
  const size_t part_floats = chunks > 1 ? static_cast<size_t>(batch) * chunks * M * panel : 0;
  const size_t bytes = (op_floats + part_floats) * sizeof(float);
  if (bytes > (6ull << 30) || M > 65535 || N > 65535 || batch * chunks > 65535) return KCG_ERR_UNSUPPORTED;
  int why = KCG_ERR_CUDA;
  float* scratch = static_cast<float*>(device_scratch(bytes, 1, stream, &why));
  if (!scratch) return why;   // the message says why (allocation failed, or growth refused during a stream capture)
  float* As = scratch;
  float* Bs = As + static_cast<size_t>(batch) * M * 3 * Kp;
  float* part = Bs + static_cast<size_t>(batch) * N * 3 * Kp;
  // A as [M rows][K]: row-major A is k-contiguous, a transposed A ([K, M]) is row-contiguous
  int rc = launch_split<0>(A, !trans_a, M, K, lda, stride_a, batch, As, Kp, kc, chunks, stream);
  if (rc) return rc;
  // B as [N rows][K]: a transposed B ([N, K]) is k-contiguous, row-major B ([K, N]) is row-contiguous
  rc = launch_split<1>(B, trans_b != 0, N, K, ldb, stride_b, batch, Bs, Kp, kc, chunks, stream);
  if (rc) return rc;
  if (chunks == 1)
    return gemm_tcgen05(KCG_F32, KCG_F32, M, N, kc3, batch, 0, 1, As, kc3, M * kc3, Bs, kc3, N * kc3, C, ldc, stride_c,
                        scale_a, scale_b, bias, act, stream, nullptr, 0);
  for (int64_t n0 = 0; n0 < N; n0 += panel) {
    const int64_t np = std::min<int64_t>(panel, N - n0);
    rc = gemm_tcgen05(KCG_F32, KCG_F32, M, np, kc3, batch * chunks, 0, 1, As, kc3, M * kc3, Bs + n0 * kc3, kc3, N * kc3, part,
                      np, M * np, nullptr, nullptr, nullptr, 0, stream, nullptr, 0);
    if (rc) return rc;
    const int64_t threads = M * ((np + 3) / 4);
    dim3 grid(static_cast<unsigned>((threads + 255) / 256), static_cast<unsigned>(batch));
    launch_overlapped(reduce_partials, grid, dim3(256), 0, stream, part, chunks, M, np, C + n0, ldc, stride_c, scale_a, scale_b,
                                              bias ? bias + n0 : nullptr, act);
    rc = check_launch("reduce_partials");
    if (rc) return rc;
  }
  return KCG_OK;
}

}  // namespace kcg
