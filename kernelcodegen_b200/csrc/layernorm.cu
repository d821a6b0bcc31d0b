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
//   ln_warp_rows   one warp per row, rows of up to 32*16 16-byte vectors, no barriers
//   ln_block_rows  one thread block per row, rows of up to 512*8 vectors
//   ln_chunk_*     rows too long (or too ragged) for the above: each row is cut
//                  into chunks, per-chunk (mean, M2) go to a scratch buffer, and a
//                  second kernel merges them (Chan's formula) and normalises.
#include "common.cuh"

#include <mutex>

namespace kcg {

void* device_scratch(size_t bytes, int slot, cudaStream_t stream, int* why);  // runtime.cu

namespace {

// Longest row (in 16-byte vectors per lane) that is given to the warp-per-row kernel (a setting
// of the calling thread).
thread_local int g_warp_row_max_vecs = 8;
// Block-per-row kernel: 16-byte vectors held by one thread (0 = chosen by row length, else 2, 4
// or 8) and rows per thread block (1, 2 or 4; negative: a persistent grid of that many blocks per
// SM); settings of the calling thread.
thread_local int g_block_vecs = 0;
thread_local int g_block_rows = 1;

// Loads, normalises and stores one row held by `nthr` cooperating threads (a warp or a
// block); `reduce` sums a float over those threads.  kExact: the row is exactly
// nthr * VPT vectors long, so no bounds checks are needed.
// kFuse: the row is not stored after normalisation but run through GELU and added to the
// matching row of `res` first, rounding to T after each step exactly where the three separate
// kernels would have stored and re-loaded it, so the result is bit-identical to the chain.
// The thread's share of a row (and, fused, of the residual row): vector i*nthr + tid for i < VPT.
template <typename T, int VPT, bool kExact, bool kFuse>
__device__ __forceinline__ void ln_row_load(const T* __restrict__ xr, const T* __restrict__ res, int tid, int nthr,
                                            int nvec, uint4 (&v)[VPT], uint4 (&rv)[kFuse ? VPT : 1]) {
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) v[i] = __ldcs(reinterpret_cast<const uint4*>(xr) + i * nthr + tid);
  // fused form: the residual row is requested together with x, so that its latency is spent
  // under the two reductions instead of after them
  if constexpr (kFuse) {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (kExact || i * nthr + tid < nvec) rv[i] = __ldcs(reinterpret_cast<const uint4*>(res) + i * nthr + tid);
  }
}

template <typename T, int VPT, bool kExact, bool kFuse, typename Reduce>
__device__ __forceinline__ void ln_row_body(const uint4 (&v)[VPT], const uint4 (&rv)[kFuse ? VPT : 1],
                                            const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ yr,
                                            int tid, int nthr, int nvec, float inv_n, float eps, Reduce reduce,
                                            float* mean_out, float* rstd_out, const uint4* g_regs = nullptr,
                                            const uint4* b_regs = nullptr, bool y_multicast = false);

template <typename T, int VPT, bool kExact, bool kFuse, typename Reduce>
__device__ __forceinline__ void ln_row(const T* __restrict__ xr, const T* __restrict__ gamma,
                                       const T* __restrict__ beta, const T* __restrict__ res, T* __restrict__ yr,
                                       int tid, int nthr, int nvec, float inv_n, float eps, Reduce reduce,
                                       float* mean_out = nullptr, float* rstd_out = nullptr, bool y_multicast = false) {
  uint4 v[VPT];
  uint4 rv[kFuse ? VPT : 1];
  ln_row_load<T, VPT, kExact, kFuse>(xr, res, tid, nthr, nvec, v, rv);
  ln_row_body<T, VPT, kExact, kFuse>(v, rv, gamma, beta, yr, tid, nthr, nvec, inv_n, eps, reduce, mean_out, rstd_out,
                                     nullptr, nullptr, y_multicast);
}

template <typename T, int VPT, bool kExact, bool kFuse, typename Reduce>
__device__ __forceinline__ void ln_row_body(const uint4 (&v)[VPT], const uint4 (&rv)[kFuse ? VPT : 1],
                                            const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ yr,
                                            int tid, int nthr, int nvec, float inv_n, float eps, Reduce reduce,
                                            float* mean_out, float* rstd_out, const uint4* g_regs,
                                            const uint4* b_regs, bool y_multicast) {
  // y_multicast: yr is an address inside an NVLink multicast mapping; the row is stored with
  // multimem.st and arrives in every bound GPU's buffer
  // g_regs / b_regs: the thread's vectors of gamma / beta already held in registers (a kernel
  // that walks over many rows loads them once); otherwise they are read here, from L1 / L2.
  using W = Words<T>;
  constexpr int EPW = W::EPW;
  // 16-bit types: the two elements of a word go through the packed fp32x2 pipe together (the
  // even and the odd elements of the thread form two partial sums that are added at the end).
  float s = 0.f;
  uint64_t s2 = 0ull;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW];
        W::unpack(w[k], f);
        if constexpr (EPW == 2) s2 = pk_add(s2, pk_make(f[0], f[1]));
        else s += f[0];
      }
    }
  if constexpr (EPW == 2) {
    float a, b;
    pk_split(s2, a, b);
    s = a + b;
  }
  const float mean = reduce(s) * inv_n;
  float q = 0.f;
  uint64_t q2 = 0ull;
  const uint64_t nmean2 = pk_make(-mean, -mean);
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) {
      const uint32_t w[4] = {opaque(v[i].x), opaque(v[i].y), opaque(v[i].z), opaque(v[i].w)};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW];
        W::unpack(w[k], f);
        if constexpr (EPW == 2) {
          const uint64_t d2 = pk_add(pk_make(f[0], f[1]), nmean2);
          q2 = pk_fma(d2, d2, q2);
        } else {
          const float d = f[0] - mean;
          q = fmaf(d, d, q);
        }
      }
    }
  if constexpr (EPW == 2) {
    float a, b;
    pk_split(q2, a, b);
    q = a + b;
  }
  const float rstd = 1.0f / sqrtf(reduce(q) * inv_n + eps);
  const float shift = -mean * rstd;
  const uint64_t rstd2 = pk_make(rstd, rstd), shift2 = pk_make(shift, shift);
  if (mean_out != nullptr && tid == 0) {  // the row's statistics, when the caller asked for them
    *mean_out = mean;
    *rstd_out = rstd;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = i * nthr + tid;
    if (kExact || vi < nvec) {
      const uint4 g4 = g_regs ? g_regs[i] : __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
      const uint4 b4 = b_regs ? b_regs[i] : __ldg(reinterpret_cast<const uint4*>(beta) + vi);
      const uint32_t w[4] = {opaque(v[i].x), opaque(v[i].y), opaque(v[i].z), opaque(v[i].w)};
      // (held in registers across rows, the packed words are made opaque so that the compiler
      // does not hoist their unpacked fp32 form out of the row loop: 128 more registers)
      const uint32_t gw[4] = {g_regs ? opaque(g4.x) : g4.x, g_regs ? opaque(g4.y) : g4.y, g_regs ? opaque(g4.z) : g4.z,
                              g_regs ? opaque(g4.w) : g4.w};
      const uint32_t bw[4] = {b_regs ? opaque(b4.x) : b4.x, b_regs ? opaque(b4.y) : b4.y, b_regs ? opaque(b4.z) : b4.z,
                              b_regs ? opaque(b4.w) : b4.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW], g[EPW], b[EPW], r[EPW];
        W::unpack(w[k], f);
        W::unpack(gw[k], g);
        W::unpack(bw[k], b);
        if constexpr (EPW == 2) {
          const uint64_t t2 = pk_fma(pk_make(f[0], f[1]), rstd2, shift2);
          pk_split(pk_fma(pk_make(g[0], g[1]), t2, pk_make(b[0], b[1])), r[0], r[1]);
        } else {
          r[0] = fmaf(g[0], fmaf(f[0], rstd, shift), b[0]);
        }
        o[k] = W::pack(r);
      }
      if constexpr (kFuse) {
        const uint4 r4 = rv[i];
        const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float y1[EPW], rs[EPW], t[EPW];
          W::unpack(o[k], y1);            // LayerNorm result as stored (rounded to T)
          W::unpack(rw[k], rs);
#pragma unroll
          for (int e = 0; e < EPW; ++e) t[e] = gelu_tanh<(sizeof(T) < 4)>(y1[e]);
          uint32_t y2w = W::pack(t);      // GELU result as stored
          W::unpack(y2w, t);
#pragma unroll
          for (int e = 0; e < EPW; ++e) t[e] = t[e] + rs[e];
          o[k] = W::pack(t);
        }
      }
      if (y_multicast) multimem_st16(reinterpret_cast<uint4*>(yr) + vi, make_uint4(o[0], o[1], o[2], o[3]));
      else __stcs(reinterpret_cast<uint4*>(yr) + vi, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// One warp per row, four rows per block, no shared memory and no block barrier; rows of
// up to 32*VPT vectors.
template <typename T, int VPT, bool kExact, bool kFuse>
__global__ void __launch_bounds__(128, 5)
ln_warp_rows(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
             const T* __restrict__ res, T* __restrict__ y, int64_t rows, int cols, float eps,
             float* __restrict__ mean_out, float* __restrict__ rstd_out, int y_multicast) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  ln_row<T, VPT, kExact, kFuse>(x + row * cols, gamma, beta, kFuse ? res + row * cols : nullptr, y + row * cols, lane, 32,
                                cols / Vec16<T>::N,
                         1.0f / static_cast<float>(cols), eps, [](float v) { return warp_sum(v); },
                         mean_out ? mean_out + row : nullptr, mean_out ? rstd_out + row : nullptr, y_multicast != 0);
}

// Sum over one group of `nthr` threads (a multiple of 32) of a block that holds several such
// groups, each working on its own row: the groups meet on their own named barrier (1 + group
// index), so a group never waits for another.  `red` is the group's own 33 floats.
__device__ __forceinline__ float group_sum(float v, float* red, int tid, int nthr, int bar_id) {
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
  v = warp_sum(v);
  if (nwarps == 1) return v;
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthr) : "memory");   // the previous call's readers are done
  if (lane == 0) red[warp] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthr) : "memory");
  const float t = lane < nwarps ? red[lane] : 0.f;
  return warp_sum(t);
}

// One group of threads per row for longer rows: `nthr` threads hold up to VPT vectors each; a
// block holds kRows such groups (kRows == 1: one thread block per row).
template <typename T, int VPT, bool kExact, bool kFuse, int kRows = 1>
__global__ void __launch_bounds__(512)
ln_block_rows(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
              const T* __restrict__ res, T* __restrict__ y, int64_t rows, int cols, float eps,
              float* __restrict__ mean_out, float* __restrict__ rstd_out, int y_multicast) {
  __shared__ float red[33 * kRows];
  grid_launch_dependents();
  grid_dependency_wait();
  if constexpr (kRows == 1) {
    const int64_t row = blockIdx.x;
    ln_row<T, VPT, kExact, kFuse>(x + row * cols, gamma, beta, kFuse ? res + row * cols : nullptr, y + row * cols,
                                  threadIdx.x, blockDim.x, cols / Vec16<T>::N, 1.0f / static_cast<float>(cols), eps,
                                  [&](float v) { return block_sum(v, red); },
                                  mean_out ? mean_out + row : nullptr, mean_out ? rstd_out + row : nullptr, y_multicast != 0);
  } else {
    const int nthr = blockDim.x / kRows;
    const int group = threadIdx.x / nthr, tid = threadIdx.x - group * nthr;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRows + group;
    if (row >= rows) return;   // whole groups leave together; the others use their own barriers
    float* my_red = red + 33 * group;
    ln_row<T, VPT, kExact, kFuse>(x + row * cols, gamma, beta, kFuse ? res + row * cols : nullptr, y + row * cols,
                                  tid, nthr, cols / Vec16<T>::N, 1.0f / static_cast<float>(cols), eps,
                                  [&](float v) { return group_sum(v, my_red, tid, nthr, 1 + group); },
                                  mean_out ? mean_out + row : nullptr, mean_out ? rstd_out + row : nullptr, y_multicast != 0);
  }
}

// Persistent form of the block-per-row kernel: a fixed grid of blocks (a few per SM) walks over
// the rows with stride gridDim.x, and a block requests its NEXT row before it starts the
// arithmetic of the current one, so that HBM latency is spent under the two reductions and the
// cost of starting and retiring a thread block is paid once per several rows.
template <typename T, int VPT, bool kExact, bool kFuse>
__global__ void __launch_bounds__(128, 2)
ln_persistent_rows(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                   const T* __restrict__ res, T* __restrict__ y, int64_t rows, int cols, float eps,
                   float* __restrict__ mean_out, float* __restrict__ rstd_out, int y_multicast) {
  __shared__ float red[33];
  grid_launch_dependents();
  grid_dependency_wait();
  const int nvec = cols / Vec16<T>::N;
  const float inv_n = 1.0f / static_cast<float>(cols);
  uint4 cur[VPT], nxt[VPT];
  uint4 rcur[kFuse ? VPT : 1], rnxt[kFuse ? VPT : 1];
  int64_t row = blockIdx.x;
  if (row >= rows) return;
  // this thread meets the same columns in every row: its share of gamma and beta stays in registers
  uint4 gq[VPT], bq[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x) < nvec) {
      gq[i] = __ldg(reinterpret_cast<const uint4*>(gamma) + i * blockDim.x + threadIdx.x);
      bq[i] = __ldg(reinterpret_cast<const uint4*>(beta) + i * blockDim.x + threadIdx.x);
    }
  ln_row_load<T, VPT, kExact, kFuse>(x + row * cols, kFuse ? res + row * cols : nullptr, threadIdx.x, blockDim.x, nvec, cur, rcur);
  for (; row < rows; row += gridDim.x) {
    const int64_t next = row + gridDim.x;
    if (next < rows)
      ln_row_load<T, VPT, kExact, kFuse>(x + next * cols, kFuse ? res + next * cols : nullptr, threadIdx.x, blockDim.x, nvec,
                                         nxt, rnxt);
    ln_row_body<T, VPT, kExact, kFuse>(cur, rcur, gamma, beta, y + row * cols, threadIdx.x, blockDim.x, nvec, inv_n, eps,
                                       [&](float v) { return block_sum(v, red); },
                                       mean_out ? mean_out + row : nullptr, mean_out ? rstd_out + row : nullptr, gq, bq,
                                       y_multicast != 0);
#pragma unroll
    for (int i = 0; i < VPT; ++i) cur[i] = nxt[i];
    if constexpr (kFuse) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) rcur[i] = rnxt[i];
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
               float eps, float* __restrict__ mean_out = nullptr, float* __restrict__ rstd_out = nullptr) {
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
  if (mean_out != nullptr && c == 0 && threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }

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
              T* y, cudaStream_t stream, const T* res = nullptr, float* mean_out = nullptr,
              float* rstd_out = nullptr, int y_mc = 0) {
  // y_mc: y is an address inside a multicast mapping (row kernels only)
  // res != nullptr: y = gelu(layernorm(x)) + res in one pass (row kernels only; the caller
  // falls back to three launches when the row kernels do not apply).
  constexpr int VW = Vec16<T>::N;
  const bool vec_ok = (cols % VW == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) &&
                      aligned16(beta) && aligned16(res);
  const int64_t nvec = cols / VW;
  const int icols = static_cast<int>(cols);
  if (rows > 0x7fffffffll * 4) return fail(KCG_ERR_UNSUPPORTED, "layernorm: more than 2^33 rows");
  if (vec_ok && nvec <= 32 * g_warp_row_max_vecs) {
    const unsigned grid = static_cast<unsigned>((rows + 3) / 4);
    const int vpt = static_cast<int>((nvec + 31) / 32);
#define KCG_LN_LAUNCH(V, E, F) launch_overlapped(ln_warp_rows<T, V, E, F>, dim3(grid), dim3(128), 0, stream, x, gamma, beta, res, y, rows, icols, eps, mean_out, rstd_out, y_mc)
#define KCG_LN_WARP(V)                                                          \
  do {                                                                          \
    const bool exact = nvec == 32 * V;                                          \
    if (res) { if (exact) KCG_LN_LAUNCH(V, true, true); else KCG_LN_LAUNCH(V, false, true); }   \
    else     { if (exact) KCG_LN_LAUNCH(V, true, false); else KCG_LN_LAUNCH(V, false, false); } \
  } while (0)
    if (vpt <= 1) KCG_LN_WARP(1);
    else if (vpt <= 2) KCG_LN_WARP(2);
    else if (vpt <= 4) KCG_LN_WARP(4);
    else if (vpt <= 8) KCG_LN_WARP(8);
    else KCG_LN_WARP(16);
#undef KCG_LN_WARP
#undef KCG_LN_LAUNCH
    return check_launch("ln_warp_rows");
  }
  // Block per row: at most 8 vectors per thread and at most 512 threads.
  if (vec_ok && nvec <= 512 * 8 && rows <= 0x7fffffffll) {
    // Vectors per thread: the setting, unless the row then needs more than 512 threads.  By default
    // rows of up to 768 vectors get 4 per thread (a bf16 row of 4096 elements is then spread over
    // 128 threads: measured 22.5 us against 23.8 us with 64 threads x 8 vectors on [8192, 4096];
    // 256 x 2, two or four rows per block and the persistent form were all slower), longer rows 8.
    int want_vpt = g_block_vecs > 0 ? g_block_vecs : (nvec <= 768 ? 4 : 8);
    while (want_vpt < 8 && (nvec + want_vpt - 1) / want_vpt > 512) want_vpt *= 2;
    int threads = static_cast<int>((nvec + want_vpt - 1) / want_vpt);
    threads = (threads + 31) / 32 * 32;
    const int vpt = static_cast<int>((nvec + threads - 1) / threads);
    if (g_block_rows < 0 && threads <= 128 && rows > static_cast<int64_t>(sm_count()) * -g_block_rows) {
      // persistent grid: -g_block_rows blocks per SM, each walking over rows
      const unsigned pgrid = static_cast<unsigned>(sm_count() * -g_block_rows);
#define KCG_LN_LAUNCH(V, E, F) launch_overlapped(ln_persistent_rows<T, V, E, F>, dim3(pgrid), dim3(threads), 0, stream, x, gamma, beta, res, y, rows, icols, eps, mean_out, rstd_out, y_mc)
#define KCG_LN_PERS(V)                                                          \
  do {                                                                          \
    const bool exact = nvec == static_cast<int64_t>(threads) * V;               \
    if (res) { if (exact) KCG_LN_LAUNCH(V, true, true); else KCG_LN_LAUNCH(V, false, true); }   \
    else     { if (exact) KCG_LN_LAUNCH(V, true, false); else KCG_LN_LAUNCH(V, false, false); } \
  } while (0)
      if (vpt <= 2) KCG_LN_PERS(2);
      else if (vpt <= 4) KCG_LN_PERS(4);
      else KCG_LN_PERS(8);
#undef KCG_LN_PERS
#undef KCG_LN_LAUNCH
      return check_launch("ln_persistent_rows");
    }
    int rpb = g_block_rows < 1 ? 1 : g_block_rows;   // rows per block, as long as the block stays within 512 threads
    while (rpb > 1 && rpb * threads > 512) rpb /= 2;
    const unsigned grid = static_cast<unsigned>((rows + rpb - 1) / rpb);
    const dim3 block(static_cast<unsigned>(threads * rpb));
#define KCG_LN_LAUNCH_R(V, E, F, R) launch_overlapped(ln_block_rows<T, V, E, F, R>, dim3(grid), block, 0, stream, x, gamma, beta, res, y, rows, icols, eps, mean_out, rstd_out, y_mc)
#define KCG_LN_LAUNCH(V, E, F)                                                  \
  do {                                                                          \
    if (rpb == 4) KCG_LN_LAUNCH_R(V, E, F, 4);                                  \
    else if (rpb == 2) KCG_LN_LAUNCH_R(V, E, F, 2);                             \
    else KCG_LN_LAUNCH_R(V, E, F, 1);                                           \
  } while (0)
#define KCG_LN_BLOCK(V)                                                         \
  do {                                                                          \
    const bool exact = nvec == static_cast<int64_t>(threads) * V;               \
    if (res) { if (exact) KCG_LN_LAUNCH(V, true, true); else KCG_LN_LAUNCH(V, false, true); }   \
    else     { if (exact) KCG_LN_LAUNCH(V, true, false); else KCG_LN_LAUNCH(V, false, false); } \
  } while (0)
    if (vpt <= 2) KCG_LN_BLOCK(2);
    else if (vpt <= 4) KCG_LN_BLOCK(4);
    else KCG_LN_BLOCK(8);
#undef KCG_LN_BLOCK
#undef KCG_LN_LAUNCH
#undef KCG_LN_LAUNCH_R
    return check_launch("ln_block_rows");
  }
  if (res || y_mc) return KCG_ERR_UNSUPPORTED;  // no fused / multicast form beyond the row kernels
  // Split-row path.
  const int64_t chunks64 = (cols + kChunk - 1) / kChunk;
  if (chunks64 > 65535 * 32 || rows > 65535)
    return fail(KCG_ERR_UNSUPPORTED,
                "layernorm: split-row path supports at most 65535 rows (got %lld) of at most "
                "%lld columns (got %lld)",
                static_cast<long long>(rows), 65535LL * 32 * kChunk, static_cast<long long>(cols));
  const int chunks = static_cast<int>(chunks64);
  int why = KCG_ERR_CUDA;
  float* stats = static_cast<float*>(device_scratch(static_cast<size_t>(rows) * chunks * 2 * sizeof(float), 0, stream, &why));
  if (!stats) return why;
  dim3 grid(chunks, static_cast<unsigned>(rows));
  ln_chunk_stats<T><<<grid, kChunkThreads, 0, stream>>>(x, stats, cols, chunks);
  int rc = check_launch("ln_chunk_stats");
  if (rc) return rc;
  ln_chunk_apply<T><<<grid, kChunkThreads, 0, stream>>>(x, gamma, beta, stats, y, cols, chunks, eps, mean_out, rstd_out);
  return check_launch("ln_chunk_apply");
}

}  // namespace
}  // namespace kcg

// ---- split-row LayerNorm without any allocation -------------------------------------------
// Scratch for kcg_layernorm_split_static(): per-(row, chunk) statistics live in this array,
// which every GPU that loads the library holds until the process exits (256 KiB).
namespace kcg {
namespace {
constexpr int64_t kStaticStatPairs = 32768;  // (row, chunk) pairs that fit
static __device__ __align__(256) float g_ln_static_stats[kStaticStatPairs * 2];

constexpr int kStaticMaxDevices = 64;
float* g_ln_static_ptr[kStaticMaxDevices] = {nullptr};
std::mutex g_ln_static_mutex;

// Device address of g_ln_static_stats on the current device.  In host code the array's
// name is only a handle, so the address is looked up once per device, with that device
// current, and cached.
int static_stats_ptr(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices)
    return fail(KCG_ERR_CUDA, "layernorm_split_static: cudaGetDevice: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(g_ln_static_mutex);
  if (!g_ln_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ln_static_stats);
    if (e != cudaSuccess || !p)
      return fail(KCG_ERR_CUDA, "layernorm_split_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_ln_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_ln_static_ptr[dev];
  return KCG_OK;
}

template <typename T>
int launch_ln_split_static(int64_t rows, int64_t cols, const T* x, const T* gamma, const T* beta, float eps, T* y,
                           cudaStream_t stream) {
  const int64_t chunks64 = (cols + kChunk - 1) / kChunk;
  if (rows > 65535 || rows * chunks64 > kStaticStatPairs)
    return fail(KCG_ERR_UNSUPPORTED,
                "layernorm_split_static: rows * ceil(cols / %d) = %lld exceeds the built-in scratch of %lld "
                "(row, chunk) pairs (and rows must not exceed 65535); use kcg_layernorm",
                kChunk, static_cast<long long>(rows * chunks64), static_cast<long long>(kStaticStatPairs));
  float* stats = nullptr;
  int rc = static_stats_ptr(&stats);
  if (rc) return rc;
  const int chunks = static_cast<int>(chunks64);
  dim3 grid(chunks, static_cast<unsigned>(rows));
  // Both kernels index stats[(row * chunks + c) * 2 + {0, 1}]; the first writes every entry
  // the second reads, so nothing has to be cleared between calls.
  ln_chunk_stats<T><<<grid, kChunkThreads, 0, stream>>>(x, stats, cols, chunks);
  rc = check_launch("ln_chunk_stats");
  if (rc) return rc;
  ln_chunk_apply<T><<<grid, kChunkThreads, 0, stream>>>(x, gamma, beta, stats, y, cols, chunks, eps);
  return check_launch("ln_chunk_apply");
}
}  // namespace
}  // namespace kcg

extern "C" int kcg_layernorm_split_static(int dtype, int64_t rows, int64_t cols, const void* x, const void* gamma,
                                          const void* beta, float eps, void* y, void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "layernorm_split_static: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !gamma || !beta || !y) return fail(KCG_ERR_INVALID_ARG, "layernorm_split_static: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KCG_F32:
      return launch_ln_split_static<float>(rows, cols, static_cast<const float*>(x), static_cast<const float*>(gamma),
                                           static_cast<const float*>(beta), eps, static_cast<float*>(y), s);
    case KCG_BF16:
      return launch_ln_split_static<__nv_bfloat16>(rows, cols, static_cast<const __nv_bfloat16*>(x),
                                                   static_cast<const __nv_bfloat16*>(gamma),
                                                   static_cast<const __nv_bfloat16*>(beta), eps,
                                                   static_cast<__nv_bfloat16*>(y), s);
    case KCG_F16:
      return launch_ln_split_static<__half>(rows, cols, static_cast<const __half*>(x), static_cast<const __half*>(gamma),
                                            static_cast<const __half*>(beta), eps, static_cast<__half*>(y), s);
    default:
      return fail(KCG_ERR_UNSUPPORTED, "layernorm_split_static: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
}

extern "C" int kcg_layernorm_gelu_add(int dtype, int64_t rows, int64_t cols, const void* x, const void* gamma,
                                      const void* beta, float eps, const void* residual, void* y, void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "layernorm_gelu_add: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !gamma || !beta || !residual || !y) return fail(KCG_ERR_INVALID_ARG, "layernorm_gelu_add: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  switch (dtype) {
    case KCG_F32:
      rc = launch_ln<float>(rows, cols, static_cast<const float*>(x), static_cast<const float*>(gamma),
                            static_cast<const float*>(beta), eps, static_cast<float*>(y), s,
                            static_cast<const float*>(residual));
      break;
    case KCG_BF16:
      rc = launch_ln<__nv_bfloat16>(rows, cols, static_cast<const __nv_bfloat16*>(x),
                                    static_cast<const __nv_bfloat16*>(gamma), static_cast<const __nv_bfloat16*>(beta),
                                    eps, static_cast<__nv_bfloat16*>(y), s, static_cast<const __nv_bfloat16*>(residual));
      break;
    case KCG_F16:
      rc = launch_ln<__half>(rows, cols, static_cast<const __half*>(x), static_cast<const __half*>(gamma),
                             static_cast<const __half*>(beta), eps, static_cast<__half*>(y), s,
                             static_cast<const __half*>(residual));
      break;
    default:
      return fail(KCG_ERR_UNSUPPORTED, "layernorm_gelu_add: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
  if (rc != KCG_ERR_UNSUPPORTED) return rc;
  // Rows the one-pass kernels do not take (too long or not vectorisable): the same three
  // operators back to back, in place in y.  That order overwrites y before the residual is
  // read, so here (unlike in the one-pass kernels) y must not overlap the residual.
  clear_error();
  {
    const size_t nbytes = static_cast<size_t>(rows) * static_cast<size_t>(cols) * kcg_dtype_size(dtype);
    const char* yb = static_cast<const char*>(y);
    const char* rb = static_cast<const char*>(residual);
    if (yb < rb + nbytes && rb < yb + nbytes)
      return fail(KCG_ERR_UNSUPPORTED,
                  "layernorm_gelu_add: rows of %lld elements run as three launches in place in y, which must then "
                  "not overlap the residual", static_cast<long long>(cols));
  }
  rc = kcg_layernorm(dtype, rows, cols, x, gamma, beta, eps, y, stream);
  if (rc) return rc;
  rc = kcg_eltwise(KCG_UNARY_GELU, dtype, dtype, rows * cols, y, y, stream);
  if (rc) return rc;
  const int64_t shape[2] = {rows, cols};
  return kcg_binary(KCG_BINARY_ADD, dtype, 2, shape, 2, shape, y, residual, y, stream);
}

extern "C" void kcg_layernorm_set_block_shape(int vecs_per_thread, int rows_per_block) {
  kcg::g_block_vecs = vecs_per_thread <= 0 ? 0 : (vecs_per_thread <= 2 ? 2 : (vecs_per_thread <= 4 ? 4 : 8));
  kcg::g_block_rows = rows_per_block < 0 ? (rows_per_block < -16 ? -16 : rows_per_block)
                                         : (rows_per_block <= 1 ? 1 : (rows_per_block <= 2 ? 2 : 4));
}

extern "C" void kcg_layernorm_set_warp_row_limit(int vecs_per_lane) {
  kcg::g_warp_row_max_vecs = vecs_per_lane < 0 ? 0 : (vecs_per_lane > 16 ? 16 : vecs_per_lane);
}

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

// ---- LayerNorm that also returns the row statistics, with optional scale / bias -----------
namespace kcg {
namespace {

template <typename T>
__global__ void fill_const(T* p, int64_t n, float value) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) p[i] = Conv<T>::from_f(value);
}

// A vector of `n` ones (slot 0) or zeros (slot 1) of element size sizeof(T), kept per device
// and grown on demand; stands in for an absent scale / bias operand so that the row kernels
// keep a single code path.  Its contents never change once written.
struct ConstVec { void* ptr = nullptr; int64_t n = 0; };
ConstVec g_const_vec[kStaticMaxDevices][3][2];
std::mutex g_const_mutex;

template <typename T>
const T* const_vector(int dtype_slot, int which, int64_t n, cudaStream_t stream) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_const_mutex);
  ConstVec& cv = g_const_vec[dev][dtype_slot][which];
  if (cv.n < n) {
    // A shorter vector handed out earlier is left allocated (launches in flight and captured
    // graphs may still read it); growing allocates, which a stream capture does not allow.
    cudaStreamCaptureStatus cap_state = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap_state) != cudaSuccess) cudaGetLastError();
    if (cap_state != cudaStreamCaptureStatusNone) return nullptr;
    cv.ptr = nullptr; cv.n = 0;
    const int64_t cap = (n + 4095) / 4096 * 4096;
    if (cudaMalloc(&cv.ptr, static_cast<size_t>(cap) * sizeof(T)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    fill_const<T><<<static_cast<unsigned>((cap + 255) / 256), 256, 0, stream>>>(static_cast<T*>(cv.ptr), cap, which == 0 ? 1.f : 0.f);
    // later calls may use other streams: make the fill visible to all of them now
    if (cudaStreamSynchronize(stream) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    cv.n = cap;
  }
  return static_cast<const T*>(cv.ptr);
}

template <typename T>
int layernorm_stats_t(int slot, int64_t rows, int64_t cols, const void* x, const void* gamma, const void* beta,
                      float eps, void* y, float* mean, float* inv_std, cudaStream_t s) {
  const T* g = static_cast<const T*>(gamma);
  const T* b = static_cast<const T*>(beta);
  if (!g) g = const_vector<T>(slot, 0, cols, s);
  if (!b) b = const_vector<T>(slot, 1, cols, s);
  if (!g || !b)
    return fail(KCG_ERR_CUDA, "layernorm_stats: could not allocate the default scale / bias vector (it cannot be "
                              "allocated while the stream is being captured: call once before the capture)");
  return launch_ln<T>(rows, cols, static_cast<const T*>(x), g, b, eps, static_cast<T*>(y), s, nullptr, mean, inv_std);
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_layernorm_stats(int dtype, int64_t rows, int64_t cols, const void* x, const void* gamma,
                                   const void* beta, float eps, void* y, float* mean, float* inv_std,
                                   void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "layernorm_stats: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !y || !mean || !inv_std) return fail(KCG_ERR_INVALID_ARG, "layernorm_stats: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KCG_F32: return layernorm_stats_t<float>(0, rows, cols, x, gamma, beta, eps, y, mean, inv_std, s);
    case KCG_BF16: return layernorm_stats_t<__nv_bfloat16>(1, rows, cols, x, gamma, beta, eps, y, mean, inv_std, s);
    case KCG_F16: return layernorm_stats_t<__half>(2, rows, cols, x, gamma, beta, eps, y, mean, inv_std, s);
    default:
      return fail(KCG_ERR_UNSUPPORTED, "layernorm_stats: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
}

// LayerNorm of a row block whose result is all-gathered by NVSwitch: every row is stored once, with
// multimem.st, to its place in a multicast mapping of all ranks' gathered tensors.
extern "C" int kcg_layernorm_allgather_multicast(int dtype, int64_t rows, int64_t cols, const void* x, const void* gamma,
                                                 const void* beta, float eps, void* gathered_multicast,
                                                 int64_t row_offset, void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0 || row_offset < 0) return fail(KCG_ERR_INVALID_ARG, "layernorm_allgather_multicast: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !gamma || !beta || !gathered_multicast) return fail(KCG_ERR_INVALID_ARG, "layernorm_allgather_multicast: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* y = static_cast<char*>(gathered_multicast) + static_cast<size_t>(row_offset) * cols * kcg_dtype_size(dtype);
  int rc;
  switch (dtype) {
    case KCG_F32:
      rc = launch_ln<float>(rows, cols, static_cast<const float*>(x), static_cast<const float*>(gamma),
                            static_cast<const float*>(beta), eps, reinterpret_cast<float*>(y), s, nullptr, nullptr, nullptr, 1);
      break;
    case KCG_BF16:
      rc = launch_ln<__nv_bfloat16>(rows, cols, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
                                    static_cast<const __nv_bfloat16*>(beta), eps, reinterpret_cast<__nv_bfloat16*>(y), s,
                                    nullptr, nullptr, nullptr, 1);
      break;
    case KCG_F16:
      rc = launch_ln<__half>(rows, cols, static_cast<const __half*>(x), static_cast<const __half*>(gamma),
                             static_cast<const __half*>(beta), eps, reinterpret_cast<__half*>(y), s, nullptr, nullptr, nullptr, 1);
      break;
    default:
      return fail(KCG_ERR_UNSUPPORTED, "layernorm_allgather_multicast: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
  if (rc == KCG_ERR_UNSUPPORTED && kcg_last_error()[0] == 0)
    return fail(KCG_ERR_UNSUPPORTED, "layernorm_allgather_multicast: rows of %lld elements are beyond the one-pass kernels "
                                     "(16-byte vectorisable rows of at most 4096 vectors)", static_cast<long long>(cols));
  return rc;
}
