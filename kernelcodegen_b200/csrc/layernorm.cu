// LayerNorm over the trailing `cols` elements of each of `rows` rows.
//
// Arithmetic follows the loop nest the reference Frontend builds for LayerNorm
// (src/Frontend/Operators.cc:1179-1243): mean = sum(x)/N, d = x - mean,
// var = sum(d*d)/N, y = gamma*(d/sqrt(var+eps)) + beta.  The reference's GPU
// schedule (src/Optimizer/Optimizer.cc:1802-1930) reads x three times and writes
// twice; these kernels read x once and write y once (a row lives in registers
// between the two reductions), which is what an HBM-bound op should cost.
//
// Three kernels:
//   ln_warp_rows   one warp per row, rows of up to 32*8 16-byte vectors, no barriers
//   ln_block_rows  one thread block per row, rows of up to 512*VPT vectors
//   ln_chunk_*     rows too long (or too ragged) for the above: each row is cut
//                  into chunks, per-chunk (mean, M2) go to a scratch buffer, and a
//                  second kernel merges them (Chan's formula) and normalises.
#include "common.cuh"

namespace kcg {

void* device_scratch(size_t bytes);  // runtime.cu

namespace {

template <typename T, int VPT>
__global__ void __launch_bounds__(256)
ln_warp_rows(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
             T* __restrict__ y, int64_t rows, int cols, float eps) {
  constexpr int VW = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int nvec = cols / VW;
  const float inv_n = 1.0f / static_cast<float>(cols);

  // gamma / beta are the same for every row: keep them in registers across the row loop
  // while they fit, otherwise re-read them (L1/L2 hits) when a row is written.
  constexpr bool kCache = VPT * (8 + VW) <= 64;
  Vec16<T> g[kCache ? VPT : 1], b[kCache ? VPT : 1];
  if constexpr (kCache) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        g[i] = ld_vec(gamma + vi * VW);
        b[i] = ld_vec(beta + vi * VW);
      }
    }
  }

  int64_t row = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5);
  const int64_t step = static_cast<int64_t>(gridDim.x) * warps;
  for (; row < rows; row += step) {
    const T* xr = x + row * cols;
    T* yr = y + row * cols;
    float v[VPT][VW];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        Vec16<T> t = ld_vec_stream(xr + vi * VW);
#pragma unroll
        for (int j = 0; j < VW; ++j) {
          v[i][j] = Conv<T>::to_f(t.v[j]);
          s += v[i][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < VW; ++j) v[i][j] = 0.f;
      }
    }
    const float mean = warp_sum(s) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < VW; ++j) {
          v[i][j] -= mean;
          q += v[i][j] * v[i][j];
        }
      }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(q) * inv_n + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * 32 + lane;
      if (vi < nvec) {
        Vec16<T> o, gg, bb;
        if constexpr (kCache) {
          gg = g[i];
          bb = b[i];
        } else {
          gg = ld_vec(gamma + vi * VW);
          bb = ld_vec(beta + vi * VW);
        }
#pragma unroll
        for (int j = 0; j < VW; ++j)
          o.v[j] = Conv<T>::from_f(Conv<T>::to_f(gg.v[j]) * (v[i][j] * rstd) + Conv<T>::to_f(bb.v[j]));
        st_vec_stream(yr + vi * VW, o);
      }
    }
  }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(512)
ln_block_rows(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
              T* __restrict__ y, int64_t rows, int cols, float eps) {
  constexpr int VW = Vec16<T>::N;
  __shared__ float red[33];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int nvec = cols / VW;
  const float inv_n = 1.0f / static_cast<float>(cols);

  // gamma / beta are the same for every row: keep them in registers across the row loop
  // while they fit, otherwise re-read them (L1/L2 hits) when a row is written.
  constexpr bool kCache = VPT * (8 + VW) <= 64;
  Vec16<T> g[kCache ? VPT : 1], b[kCache ? VPT : 1];
  if constexpr (kCache) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * nthr + tid;
      if (vi < nvec) {
        g[i] = ld_vec(gamma + vi * VW);
        b[i] = ld_vec(beta + vi * VW);
      }
    }
  }

  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    T* yr = y + row * cols;
    float v[VPT][VW];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * nthr + tid;
      if (vi < nvec) {
        Vec16<T> t = ld_vec_stream(xr + vi * VW);
#pragma unroll
        for (int j = 0; j < VW; ++j) {
          v[i][j] = Conv<T>::to_f(t.v[j]);
          s += v[i][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < VW; ++j) v[i][j] = 0.f;
      }
    }
    const float mean = block_sum(s, red) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * nthr + tid;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < VW; ++j) {
          v[i][j] -= mean;
          q += v[i][j] * v[i][j];
        }
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) * inv_n + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = i * nthr + tid;
      if (vi < nvec) {
        Vec16<T> o, gg, bb;
        if constexpr (kCache) {
          gg = g[i];
          bb = b[i];
        } else {
          gg = ld_vec(gamma + vi * VW);
          bb = ld_vec(beta + vi * VW);
        }
#pragma unroll
        for (int j = 0; j < VW; ++j)
          o.v[j] = Conv<T>::from_f(Conv<T>::to_f(gg.v[j]) * (v[i][j] * rstd) + Conv<T>::to_f(bb.v[j]));
        st_vec_stream(yr + vi * VW, o);
      }
    }
  }
}

// ---- split-row path ----------------------------------------------------------------
// A chunk is kChunk consecutive elements of one row (the last chunk may be short).
constexpr int kChunk = 8192;
constexpr int kChunkThreads = 256;
constexpr int kChunkPerThread = kChunk / kChunkThreads;  // 32

// stats[(row*chunks + c)*2 + 0] = mean of the chunk, [+1] = sum of squared deviations.
template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
ln_chunk_stats(const T* __restrict__ x, float* __restrict__ stats, int64_t cols, int chunks) {
  __shared__ float red[33];
  const int c = blockIdx.x;
  const int64_t row = blockIdx.y;
  const int64_t base = static_cast<int64_t>(c) * kChunk;
  const int len = static_cast<int>(min(static_cast<int64_t>(kChunk), cols - base));
  const T* xr = x + row * cols + base;
  float v[kChunkPerThread];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kChunkPerThread; ++i) {
    const int e = i * kChunkThreads + threadIdx.x;
    v[i] = (e < len) ? Conv<T>::to_f(xr[e]) : 0.f;
    s += v[i];
  }
  const float mean = block_sum(s, red) / static_cast<float>(len);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < kChunkPerThread; ++i) {
    const int e = i * kChunkThreads + threadIdx.x;
    if (e < len) {
      const float d = v[i] - mean;
      q += d * d;
    }
  }
  q = block_sum(q, red);
  if (threadIdx.x == 0) {
    float* o = stats + (row * chunks + c) * 2;
    o[0] = mean;
    o[1] = q;
  }
}

template <typename T>
__global__ void __launch_bounds__(kChunkThreads)
ln_chunk_apply(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
               const float* __restrict__ stats, T* __restrict__ y, int64_t cols, int chunks,
               float eps) {
  __shared__ float red[33];
  const int c = blockIdx.x;
  const int64_t row = blockIdx.y;
  const float* st = stats + row * chunks * 2;
  // Merge the per-chunk statistics of this row: mean = sum(n_c*mean_c)/N,
  // M2 = sum(M2_c) + sum(n_c*(mean_c-mean)^2).
  float wsum = 0.f;
  for (int k = threadIdx.x; k < chunks; k += kChunkThreads) {
    const float n_c = static_cast<float>(min(static_cast<int64_t>(kChunk), cols - static_cast<int64_t>(k) * kChunk));
    wsum += n_c * st[2 * k];
  }
  const float n_all = static_cast<float>(cols);
  const float mean = block_sum(wsum, red) / n_all;
  float m2 = 0.f;
  for (int k = threadIdx.x; k < chunks; k += kChunkThreads) {
    const float n_c = static_cast<float>(min(static_cast<int64_t>(kChunk), cols - static_cast<int64_t>(k) * kChunk));
    const float d = st[2 * k] - mean;
    m2 += st[2 * k + 1] + n_c * d * d;
  }
  const float rstd = 1.0f / sqrtf(block_sum(m2, red) / n_all + eps);

  const int64_t base = static_cast<int64_t>(c) * kChunk;
  const int len = static_cast<int>(min(static_cast<int64_t>(kChunk), cols - base));
  const T* xr = x + row * cols + base;
  T* yr = y + row * cols + base;
  const T* gr = gamma + base;
  const T* br = beta + base;
#pragma unroll 4
  for (int i = 0; i < kChunkPerThread; ++i) {
    const int e = i * kChunkThreads + threadIdx.x;
    if (e < len) {
      const float d = Conv<T>::to_f(xr[e]) - mean;
      yr[e] = Conv<T>::from_f(Conv<T>::to_f(gr[e]) * (d * rstd) + Conv<T>::to_f(br[e]));
    }
  }
}

template <typename T>
int launch_ln(int64_t rows, int64_t cols, const T* x, const T* gamma, const T* beta, float eps,
              T* y, cudaStream_t stream) {
  constexpr int VW = Vec16<T>::N;
  const bool vec_ok = (cols % VW == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) &&
                      aligned16(beta);
  const int64_t nvec = cols / VW;
  const int sms = sm_count();
  if (vec_ok && nvec <= 32 * 8) {
    const int warps = 8;
    const int64_t want = (rows + warps - 1) / warps;
    const int grid = static_cast<int>(want < static_cast<int64_t>(sms) * 8 ? want : static_cast<int64_t>(sms) * 8);
    const int vpt = static_cast<int>((nvec + 31) / 32);
#define KCG_LN_WARP(V)                                                                   \
  ln_warp_rows<T, V><<<grid, warps * 32, 0, stream>>>(x, gamma, beta, y, rows,           \
                                                      static_cast<int>(cols), eps)
    if (vpt <= 1) KCG_LN_WARP(1);
    else if (vpt <= 2) KCG_LN_WARP(2);
    else if (vpt <= 4) KCG_LN_WARP(4);
    else KCG_LN_WARP(8);
#undef KCG_LN_WARP
    return check_launch("ln_warp_rows");
  }
  // Block per row while a row fits 512 threads x (64 fp32 values per thread).
  constexpr int kMaxVpt = 64 / VW;
  if (vec_ok && nvec <= 512 * kMaxVpt) {
    // Aim for at most 256 threads; widen per-thread work first, then the block.
    int vpt = 1;
    while (vpt < kMaxVpt && nvec > 256 * vpt) vpt *= 2;
    int threads = static_cast<int>((nvec + vpt - 1) / vpt);
    threads = (threads + 31) / 32 * 32;
    const int ctas_per_sm = 2048 / threads > 8 ? 8 : 2048 / threads;
    const int64_t cap = static_cast<int64_t>(sms) * (ctas_per_sm > 0 ? ctas_per_sm : 1);
    const int grid = static_cast<int>(rows < cap ? rows : cap);
#define KCG_LN_BLOCK(V)                                                                  \
  ln_block_rows<T, V><<<grid, threads, 0, stream>>>(x, gamma, beta, y, rows,             \
                                                    static_cast<int>(cols), eps)
    switch (vpt) {
      case 1: KCG_LN_BLOCK(1); break;
      case 2: KCG_LN_BLOCK(2); break;
      case 4: KCG_LN_BLOCK(4); break;
      case 8: if constexpr (kMaxVpt >= 8) { KCG_LN_BLOCK(8); } break;
      case 16: if constexpr (kMaxVpt >= 16) { KCG_LN_BLOCK(16); } break;
      default: return fail(KCG_ERR_UNSUPPORTED, "layernorm: unexpected vectors per thread %d", vpt);
    }
#undef KCG_LN_BLOCK
    return check_launch("ln_block_rows");
  }
  // Split-row path.
  const int64_t chunks64 = (cols + kChunk - 1) / kChunk;
  if (chunks64 > 65535 * 32 || rows > 65535)
    return fail(KCG_ERR_UNSUPPORTED,
                "layernorm: split-row path supports at most 65535 rows (got %lld) of at most "
                "%lld columns (got %lld)",
                static_cast<long long>(rows), 65535LL * 32 * kChunk, static_cast<long long>(cols));
  const int chunks = static_cast<int>(chunks64);
  float* stats = static_cast<float*>(device_scratch(static_cast<size_t>(rows) * chunks * 2 * sizeof(float)));
  if (!stats) return fail(KCG_ERR_CUDA, "layernorm: could not allocate %zu bytes of scratch",
                          static_cast<size_t>(rows) * chunks * 2 * sizeof(float));
  dim3 grid(chunks, static_cast<unsigned>(rows));
  ln_chunk_stats<T><<<grid, kChunkThreads, 0, stream>>>(x, stats, cols, chunks);
  int rc = check_launch("ln_chunk_stats");
  if (rc) return rc;
  ln_chunk_apply<T><<<grid, kChunkThreads, 0, stream>>>(x, gamma, beta, stats, y, cols, chunks, eps);
  return check_launch("ln_chunk_apply");
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_layernorm(int dtype, int64_t rows, int64_t cols, const void* x,
                             const void* gamma, const void* beta, float eps, void* y,
                             void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "layernorm: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !gamma || !beta || !y) return fail(KCG_ERR_INVALID_ARG, "layernorm: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KCG_F32:
      return launch_ln<float>(rows, cols, static_cast<const float*>(x),
                              static_cast<const float*>(gamma), static_cast<const float*>(beta),
                              eps, static_cast<float*>(y), s);
    case KCG_BF16:
      return launch_ln<__nv_bfloat16>(rows, cols, static_cast<const __nv_bfloat16*>(x),
                                      static_cast<const __nv_bfloat16*>(gamma),
                                      static_cast<const __nv_bfloat16*>(beta), eps,
                                      static_cast<__nv_bfloat16*>(y), s);
    case KCG_F16:
      return launch_ln<__half>(rows, cols, static_cast<const __half*>(x),
                               static_cast<const __half*>(gamma), static_cast<const __half*>(beta),
                               eps, static_cast<__half*>(y), s);
    default:
      return fail(KCG_ERR_UNSUPPORTED, "layernorm: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
}
