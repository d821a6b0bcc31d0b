// fp32 GEMM on the CUDA cores.
//
// The reference's only shipped GEMM is fp32 FFMA code (schedule:
// src/Optimizer/Optimizer.cc:406-570 — 128x128x8 CTA tile, 8x8 per thread), and the
// fp32 configuration is held to a relative error of 1e-5, which tensor cores cannot
// deliver for fp32 inputs (tf32 keeps 10 mantissa bits).  So fp32 stays on FFMA with
// the reference's own accumulation order: each C element is a single fp32 accumulator
// that starts at 0 and receives a*b in increasing k (src/Frontend/Operators.cc:186-213).
// Unlike the reference kernel this one takes any M, N, K, both operand layouts and a
// batch dimension.
#include "common.cuh"

namespace kcg {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, PAD = 4;

struct SgemmArgs {
  const float* A; const float* B; float* C;
  int64_t M, N, K;
  int64_t a_sm, a_sk;  // element strides of A(m,k)
  int64_t b_sk, b_sn;  // element strides of B(k,n)
  int64_t ldc;
  int64_t batch_a, batch_b, batch_c;
  const float* scale_a; const float* scale_b;
  const float* bias; int act;
};

// kAK: A is contiguous along k (row-major [M,K]); otherwise contiguous along m.
// kBN: B is contiguous along n (row-major [K,N]); otherwise contiguous along k.
template <bool kAK, bool kBN>
__global__ void __launch_bounds__(256) sgemm_kernel(const SgemmArgs p) {
  __shared__ __align__(16) float As[2][BK][BM + PAD];
  __shared__ __align__(16) float Bs[2][BK][BN + PAD];
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * BN;
  const float* A = p.A + blockIdx.z * p.batch_a;
  const float* B = p.B + blockIdx.z * p.batch_b;
  float* C = p.C + blockIdx.z * p.batch_c;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float ra[8], rb[8];
  auto load_tiles = [&](int64_t k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int m, k;
      if (kAK) { k = t & 15; m = (t >> 4) + 16 * i; }
      else     { m = t & 127; k = (t >> 7) + 2 * i; }
      const int64_t gm = m0 + m, gk = k0 + k;
      ra[i] = (gm < p.M && gk < p.K) ? A[gm * p.a_sm + gk * p.a_sk] : 0.f;
      int n, kb;
      if (kBN) { n = t & 127; kb = (t >> 7) + 2 * i; }
      else     { kb = t & 15; n = (t >> 4) + 16 * i; }
      const int64_t gn = n0 + n, gkb = k0 + kb;
      rb[i] = (gn < p.N && gkb < p.K) ? B[gkb * p.b_sk + gn * p.b_sn] : 0.f;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int m, k;
      if (kAK) { k = t & 15; m = (t >> 4) + 16 * i; }
      else     { m = t & 127; k = (t >> 7) + 2 * i; }
      As[buf][k][m] = ra[i];
      int n, kb;
      if (kBN) { n = t & 127; kb = (t >> 7) + 2 * i; }
      else     { kb = t & 15; n = (t >> 4) + 16 * i; }
      Bs[buf][kb][n] = rb[i];
    }
  };

  const int64_t ktiles = (p.K + BK - 1) / BK;
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  for (int64_t kt = 0; kt < ktiles; ++kt) {
    const int buf = static_cast<int>(kt & 1);
    if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[8], b[8];
      *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      *reinterpret_cast<float4*>(&a[4]) = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      *reinterpret_cast<float4*>(&b[4]) = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) {
      store_tiles(buf ^ 1);
      __syncthreads();
    }
  }

  float alpha = 1.f;
  if (p.scale_a) alpha *= *p.scale_a;
  if (p.scale_b) alpha *= *p.scale_b;
  const bool vec = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= p.M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int64_t gn = n0 + jh * 64 + tx * 4;
      float* dst = C + gm * p.ldc + gn;
      if (vec && gn + 3 < p.N) {
        float4 o = make_float4(gemm_epilogue_value<float>(acc[i][jh * 4 + 0], alpha, p.bias, gn + 0, p.act),
                               gemm_epilogue_value<float>(acc[i][jh * 4 + 1], alpha, p.bias, gn + 1, p.act),
                               gemm_epilogue_value<float>(acc[i][jh * 4 + 2], alpha, p.bias, gn + 2, p.act),
                               gemm_epilogue_value<float>(acc[i][jh * 4 + 3], alpha, p.bias, gn + 3, p.act));
        *reinterpret_cast<float4*>(dst) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (gn + j < p.N) dst[j] = gemm_epilogue_value<float>(acc[i][jh * 4 + j], alpha, p.bias, gn + j, p.act);
      }
    }
  }
}

}  // namespace

int sgemm_f32(int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a, int trans_b,
              const float* A, int64_t lda, int64_t stride_a, const float* B, int64_t ldb,
              int64_t stride_b, float* C, int64_t ldc, int64_t stride_c, const float* scale_a,
              const float* scale_b, const float* bias, int act, cudaStream_t stream) {
  SgemmArgs p;
  p.A = A; p.B = B; p.C = C; p.M = M; p.N = N; p.K = K;
  if (!trans_a) { p.a_sm = lda; p.a_sk = 1; } else { p.a_sm = 1; p.a_sk = lda; }
  if (!trans_b) { p.b_sk = ldb; p.b_sn = 1; } else { p.b_sk = 1; p.b_sn = ldb; }
  p.ldc = ldc; p.batch_a = stride_a; p.batch_b = stride_b; p.batch_c = stride_c;
  p.scale_a = scale_a; p.scale_b = scale_b; p.bias = bias; p.act = act;
  const int64_t gx = (N + BN - 1) / BN, gy = (M + BM - 1) / BM;
  if (gy > 65535 || batch > 65535)
    return fail(KCG_ERR_UNSUPPORTED, "fp32 gemm: M/128 and batch must not exceed 65535");
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
  if (!trans_a && !trans_b) sgemm_kernel<true, true><<<grid, 256, 0, stream>>>(p);
  else if (!trans_a && trans_b) sgemm_kernel<true, false><<<grid, 256, 0, stream>>>(p);
  else if (trans_a && !trans_b) sgemm_kernel<false, true><<<grid, 256, 0, stream>>>(p);
  else sgemm_kernel<false, false><<<grid, 256, 0, stream>>>(p);
  return check_launch("sgemm_kernel");
}

}  // namespace kcg
