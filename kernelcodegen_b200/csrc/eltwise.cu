// Unary maps, binary maps with broadcasting, and the row softmax.
//
// Definitions follow the reference Frontend: unary ops
// src/Frontend/Operators.cc:960-1000 (Gelu with the literal constants 0.797884 and
// 0.044715), Relu :222-289, binary ops and the broadcast rule :581-612 and :772-889,
// softmax :462-578.  The reference schedules (src/Optimizer/Optimizer.cc:928-1175)
// tile a near-square 2-D view 64x64 with 4x4 elements per thread; here every map is a
// flat stream of 128-bit accesses, because the ops are HBM-bound and have no reuse.
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace kcg {
namespace {

// ---------------------------------------------------------------- unary functors
// kFast selects hardware approximations whose error is below the rounding of a
// 16-bit result; fp32 results use the accurate library routines.
template <bool kFast> __device__ __forceinline__ float tanh_f(float v) {
  if constexpr (kFast) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
  } else {
    return tanhf(v);
  }
}

struct OpTanh { template <bool F> static __device__ __forceinline__ float f(float v) { return tanh_f<F>(v); } };
struct OpSqrt { template <bool F> static __device__ __forceinline__ float f(float v) { return sqrtf(v); } };
struct OpLog  { template <bool F> static __device__ __forceinline__ float f(float v) { return F ? __logf(v) : logf(v); } };
struct OpRelu { template <bool F> static __device__ __forceinline__ float f(float v) { return fmaxf(0.f, v); } };
struct OpCast { template <bool F> static __device__ __forceinline__ float f(float v) { return v; } };
struct OpGelu { template <bool F> static __device__ __forceinline__ float f(float v) { return gelu_tanh<F>(v); } };

template <typename TI, typename TO, typename Op, int UNROLL>
__global__ void __launch_bounds__(256)
unary_vec(const TI* __restrict__ x, TO* __restrict__ y, int64_t ngroups, bool wide32) {
  // One group = EPT elements = whole 16-byte vectors on both sides.
  constexpr int EPT = 16 / (sizeof(TI) < sizeof(TO) ? sizeof(TI) : sizeof(TO));
  constexpr int NI = EPT * sizeof(TI) / 16, NO = EPT * sizeof(TO) / 16;
  constexpr bool kFast = sizeof(TO) < 4;
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * blockDim.x * UNROLL + threadIdx.x;
  for (; g0 < ngroups; g0 += stride * UNROLL) {
    Vec16<TI> in[UNROLL][NI];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t g = g0 + static_cast<int64_t>(u) * blockDim.x;
      if (g < ngroups) {
        if constexpr (NI == 2) {
          if (wide32) {
            ld_256(x + g * EPT, *reinterpret_cast<uint4*>(&in[u][0]), *reinterpret_cast<uint4*>(&in[u][1]));
            continue;
          }
        }
#pragma unroll
        for (int k = 0; k < NI; ++k) in[u][k] = ld_vec_stream(x + g * EPT + k * Vec16<TI>::N);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t g = g0 + static_cast<int64_t>(u) * blockDim.x;
      if (g < ngroups) {
        Vec16<TO> out[NO];
        if constexpr (std::is_same<Op, OpGelu>::value && kFast && EPT % 2 == 0) {
          // two elements per step on the packed fp32x2 pipe (same bits as the scalar form)
#pragma unroll
          for (int e = 0; e < EPT; e += 2) {
            float v0 = Conv<TI>::to_f(in[u][e / Vec16<TI>::N].v[e % Vec16<TI>::N]);
            float v1 = Conv<TI>::to_f(in[u][(e + 1) / Vec16<TI>::N].v[(e + 1) % Vec16<TI>::N]);
            gelu_tanh_pair<true>(v0, v1);
            out[e / Vec16<TO>::N].v[e % Vec16<TO>::N] = Conv<TO>::from_f(v0);
            out[(e + 1) / Vec16<TO>::N].v[(e + 1) % Vec16<TO>::N] = Conv<TO>::from_f(v1);
          }
        } else {
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
          const float v = Conv<TI>::to_f(in[u][e / Vec16<TI>::N].v[e % Vec16<TI>::N]);
          out[e / Vec16<TO>::N].v[e % Vec16<TO>::N] = Conv<TO>::from_f(Op::template f<kFast>(v));
        }
        }
        if constexpr (NO == 2) {
          if (wide32) {
            st_256(y + g * EPT, *reinterpret_cast<const uint4*>(&out[0]), *reinterpret_cast<const uint4*>(&out[1]));
            continue;
          }
        }
#pragma unroll
        for (int k = 0; k < NO; ++k) st_vec_stream(y + g * EPT + k * Vec16<TO>::N, out[k]);
      }
    }
  }
}

template <typename TI, typename TO, typename Op>
__global__ void __launch_bounds__(256)
unary_scalar(const TI* __restrict__ x, TO* __restrict__ y, int64_t begin, int64_t n) {
  constexpr bool kFast = sizeof(TO) < 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = Conv<TO>::from_f(Op::template f<kFast>(Conv<TI>::to_f(x[i])));
}

template <typename TI, typename TO, typename Op>
int launch_unary(int64_t n, const void* xv, void* yv, cudaStream_t stream) {
  const TI* x = static_cast<const TI*>(xv);
  TO* y = static_cast<TO*>(yv);
  constexpr int EPT = 16 / (sizeof(TI) < sizeof(TO) ? sizeof(TI) : sizeof(TO));
  constexpr int UNROLL = 4;
  const int sms = sm_count();
  int64_t done = 0;
  if (aligned16(x) && aligned16(y) && n >= EPT) {
    const int64_t ngroups = n / EPT;
    const int64_t want = (ngroups + 256 * UNROLL - 1) / (256 * UNROLL);
    const int64_t cap = static_cast<int64_t>(sms) * 8;
    launch_overlapped(unary_vec<TI, TO, Op, UNROLL>, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0, stream,
                      x, y, ngroups, (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && (reinterpret_cast<uintptr_t>(y) & 31u) == 0);
    int rc = check_launch("unary_vec");
    if (rc) return rc;
    done = ngroups * EPT;
  }
  if (done < n) {
    const int64_t rest = n - done;
    const int64_t want = (rest + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sms) * 8;
    unary_scalar<TI, TO, Op><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(x, y, done, n);
    return check_launch("unary_scalar");
  }
  return KCG_OK;
}

template <typename T, typename Op>
int unary_same(int dtype, int64_t n, const void* x, void* y, cudaStream_t s);

template <typename Op>
int dispatch_unary_same(int dtype, int64_t n, const void* x, void* y, cudaStream_t s) {
  switch (dtype) {
    case KCG_F32: return launch_unary<float, float, Op>(n, x, y, s);
    case KCG_BF16: return launch_unary<__nv_bfloat16, __nv_bfloat16, Op>(n, x, y, s);
    case KCG_F16: return launch_unary<__half, __half, Op>(n, x, y, s);
    default: return fail(KCG_ERR_UNSUPPORTED, "eltwise: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
}

template <typename TI>
int dispatch_cast_out(int dtype_out, int64_t n, const void* x, void* y, cudaStream_t s) {
  switch (dtype_out) {
    case KCG_F32: return launch_unary<TI, float, OpCast>(n, x, y, s);
    case KCG_BF16: return launch_unary<TI, __nv_bfloat16, OpCast>(n, x, y, s);
    case KCG_F16: return launch_unary<TI, __half, OpCast>(n, x, y, s);
    case KCG_I32: return launch_unary<TI, int32_t, OpCast>(n, x, y, s);
    default: return fail(KCG_ERR_UNSUPPORTED, "eltwise Cast: target dtype %d has no kernel", dtype_out);
  }
}

// ---------------------------------------------------------------- binary functors
struct BAdd { static __device__ __forceinline__ float f(float a, float b) { return a + b; } };
struct BMul { static __device__ __forceinline__ float f(float a, float b) { return a * b; } };
struct BDiv { static __device__ __forceinline__ float f(float a, float b) { return a / b; } };
struct BSub { static __device__ __forceinline__ float f(float a, float b) { return a - b; } };
struct BPow { static __device__ __forceinline__ float f(float a, float b) { return powf(a, b); } };
struct BEq  { static __device__ __forceinline__ float f(float a, float b) { return a == b ? 1.f : 0.f; } };
struct BGt  { static __device__ __forceinline__ float f(float a, float b) { return a > b ? 1.f : 0.f; } };

// Both operands have the output shape.
template <typename T, typename Op, int UNROLL>
__global__ void __launch_bounds__(256)
binary_same_vec(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c, int64_t nvec) {
  constexpr int VW = Vec16<T>::N;
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * blockDim.x * UNROLL + threadIdx.x;
  for (; g0 < nvec; g0 += stride * UNROLL) {
    Vec16<T> va[UNROLL], vb[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t g = g0 + static_cast<int64_t>(u) * blockDim.x;
      if (g < nvec) {
        va[u] = ld_vec_stream(a + g * VW);
        vb[u] = ld_vec_stream(b + g * VW);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t g = g0 + static_cast<int64_t>(u) * blockDim.x;
      if (g < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < VW; ++j)
          o.v[j] = Conv<T>::from_f(Op::f(Conv<T>::to_f(va[u].v[j]), Conv<T>::to_f(vb[u].v[j])));
        st_vec_stream(c + g * VW, o);
      }
    }
  }
}

// General broadcast.  Dimensions are collapsed on the host; dim 0 is innermost.
struct BcastDims {
  int rank;
  int64_t extent[KCG_MAX_RANK];
  int64_t stride_a[KCG_MAX_RANK];  // 0 where a is broadcast
  int64_t stride_b[KCG_MAX_RANK];
};

// Each thread produces VEC consecutive outputs along the innermost dimension
// (extent[0] % VEC == 0).  An operand whose inner stride is 1 is read as a vector
// when VEC is a whole 16-byte vector; one whose inner stride is 0 is read once.
template <typename T, typename Op, int VEC>
__global__ void __launch_bounds__(256)
binary_bcast(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
             const BcastDims d, int64_t ngroups) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t inner_groups = d.extent[0] / VEC;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < ngroups; g += stride) {
    int64_t rem = g / inner_groups;
    const int64_t i0 = (g % inner_groups) * VEC;
    int64_t oa = i0 * d.stride_a[0], ob = i0 * d.stride_b[0];
#pragma unroll 1
    for (int k = 1; k < d.rank; ++k) {
      const int64_t idx = rem % d.extent[k];
      rem /= d.extent[k];
      oa += idx * d.stride_a[k];
      ob += idx * d.stride_b[k];
    }
    float fa[VEC], fb[VEC];
    if constexpr (VEC == Vec16<T>::N) {
      if (d.stride_a[0] == 1) {
        Vec16<T> t = ld_vec(a + oa);
#pragma unroll
        for (int j = 0; j < VEC; ++j) fa[j] = Conv<T>::to_f(t.v[j]);
      } else {
        const float s = Conv<T>::to_f(a[oa]);
#pragma unroll
        for (int j = 0; j < VEC; ++j) fa[j] = s;
      }
      if (d.stride_b[0] == 1) {
        Vec16<T> t = ld_vec(b + ob);
#pragma unroll
        for (int j = 0; j < VEC; ++j) fb[j] = Conv<T>::to_f(t.v[j]);
      } else {
        const float s = Conv<T>::to_f(b[ob]);
#pragma unroll
        for (int j = 0; j < VEC; ++j) fb[j] = s;
      }
      Vec16<T> o;
#pragma unroll
      for (int j = 0; j < VEC; ++j) o.v[j] = Conv<T>::from_f(Op::f(fa[j], fb[j]));
      st_vec(c + g * VEC, o);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        fa[j] = Conv<T>::to_f(a[oa + j * d.stride_a[0]]);
        fb[j] = Conv<T>::to_f(b[ob + j * d.stride_b[0]]);
        c[g * VEC + j] = Conv<T>::from_f(Op::f(fa[j], fb[j]));
      }
    }
  }
}

// The bias-shaped broadcast: one operand has the full [rows, inner] shape, the other is an
// `inner`-long vector repeated over the rows (any number of leading broadcast dims collapse to
// this).  A thread keeps its 16-byte piece of the vector in registers and walks down the rows, so
// the full operand streams with no index arithmetic; kSwap: the vector is the left operand.
template <typename T, typename Op, bool kSwap, int UNROLL>
__global__ void __launch_bounds__(256)
binary_row_vector(const T* __restrict__ full, const T* __restrict__ vec, T* __restrict__ c, int64_t rows,
                  int64_t inner_vecs) {
  constexpr int VW = Vec16<T>::N;
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= inner_vecs) return;
  const Vec16<T> vv = ld_vec(vec + j * VW);
  float fv[VW];
#pragma unroll
  for (int e = 0; e < VW; ++e) fv[e] = Conv<T>::to_f(vv.v[e]);
  const int64_t pitch = inner_vecs * VW;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.y) * UNROLL; r0 < rows; r0 += static_cast<int64_t>(gridDim.y) * UNROLL) {
    Vec16<T> in[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (r0 + u < rows) in[u] = ld_vec_stream(full + (r0 + u) * pitch + j * VW);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (r0 + u < rows) {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < VW; ++e) {
          const float x = Conv<T>::to_f(in[u].v[e]);
          o.v[e] = Conv<T>::from_f(kSwap ? Op::f(fv[e], x) : Op::f(x, fv[e]));
        }
        st_vec_stream(c + (r0 + u) * pitch + j * VW, o);
      }
  }
}

template <typename T, typename Op>
int launch_binary(const BcastDims& d, bool same_shape, int64_t total, const void* av,
                  const void* bv, void* cv, cudaStream_t stream) {
  const T* a = static_cast<const T*>(av);
  const T* b = static_cast<const T*>(bv);
  T* c = static_cast<T*>(cv);
  constexpr int VW = Vec16<T>::N;
  const int sms = sm_count();
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  const bool al = aligned16(a) && aligned16(b) && aligned16(c);
  if (same_shape && al && total % VW == 0) {
    constexpr int UNROLL = 4;
    const int64_t nvec = total / VW;
    const int64_t want = (nvec + 256 * UNROLL - 1) / (256 * UNROLL);
    launch_overlapped(binary_same_vec<T, Op, UNROLL>, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0, stream,
                      a, b, c, nvec);
    return check_launch("binary_same_vec");
  }
  // Vector accesses along the innermost dimension need every outer stride to keep
  // 16-byte alignment, which holds when the inner extent is a multiple of VW.
  bool vec_ok = al && d.extent[0] % VW == 0;
  for (int k = 1; k < d.rank && vec_ok; ++k)
    vec_ok = (d.stride_a[k] % VW == 0) && (d.stride_b[k] % VW == 0);
  // [rows, inner] (op) [inner] in either order
  if (vec_ok && d.rank == 2 && d.stride_a[0] == 1 && d.stride_b[0] == 1 &&
      ((d.stride_a[1] == d.extent[0] && d.stride_b[1] == 0) || (d.stride_b[1] == d.extent[0] && d.stride_a[1] == 0))) {
    constexpr int UNROLL = 4;
    const bool swap = d.stride_a[1] == 0;   // the vector is the left operand
    const int64_t inner_vecs = d.extent[0] / VW, rows = d.extent[1];
    const int64_t gx = (inner_vecs + 255) / 256;
    int64_t gy = (rows + UNROLL - 1) / UNROLL;
    const int64_t gy_cap = std::max<int64_t>(1, cap * 2 / gx);
    if (gy > gy_cap) gy = gy_cap;
    if (gx <= 0x7fffffffll && gy <= 65535) {
      dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
      if (swap) launch_overlapped(binary_row_vector<T, Op, true, UNROLL>, grid, dim3(256), 0, stream, b, a, c, rows, inner_vecs);
      else launch_overlapped(binary_row_vector<T, Op, false, UNROLL>, grid, dim3(256), 0, stream, a, b, c, rows, inner_vecs);
      return check_launch("binary_row_vector");
    }
  }
  if (vec_ok) {
    const int64_t ngroups = total / VW;
    const int64_t want = (ngroups + 255) / 256;
    binary_bcast<T, Op, VW><<<static_cast<int>(want < cap * 4 ? want : cap * 4), 256, 0, stream>>>(a, b, c, d, ngroups);
  } else {
    const int64_t want = (total + 255) / 256;
    binary_bcast<T, Op, 1><<<static_cast<int>(want < cap * 4 ? want : cap * 4), 256, 0, stream>>>(a, b, c, d, total);
  }
  return check_launch("binary_bcast");
}

template <typename Op>
int dispatch_binary_dtype(int dtype, const BcastDims& d, bool same, int64_t total, const void* a,
                          const void* b, void* c, cudaStream_t s) {
  switch (dtype) {
    case KCG_F32: return launch_binary<float, Op>(d, same, total, a, b, c, s);
    case KCG_BF16: return launch_binary<__nv_bfloat16, Op>(d, same, total, a, b, c, s);
    case KCG_F16: return launch_binary<__half, Op>(d, same, total, a, b, c, s);
    default: return fail(KCG_ERR_UNSUPPORTED, "binary: dtype %d has no kernel (float32, bfloat16, float16)", dtype);
  }
}

// ---------------------------------------------------------------- softmax
// One thread block per row, the row is read twice (max+sum online, then normalise);
// the second read of a row that was just streamed is served from L2.
template <typename T>
__global__ void __launch_bounds__(256)
softmax_rows(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols, float scale,
             int causal, int64_t q_len) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    T* yr = y + row * cols;
    int64_t valid = cols;
    if (causal) {
      const int64_t i = row % q_len;
      valid = i + (cols - q_len) + 1;
      if (valid > cols) valid = cols;
      if (valid < 0) valid = 0;
    }
    float m = -INFINITY, s = 0.f;
    for (int64_t j = threadIdx.x; j < valid; j += blockDim.x) {
      const float v = Conv<T>::to_f(xr[j]) * scale;
      const float nm = fmaxf(m, v);
      s = s * __expf(m - nm) + __expf(v - nm);
      m = nm;
    }
    const float gm = block_max(m, red);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum(s, red);
    const float inv = gs > 0.f ? 1.0f / gs : 0.f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
      float o = 0.f;
      if (j < valid) o = __expf(Conv<T>::to_f(xr[j]) * scale - gm) * inv;
      yr[j] = Conv<T>::from_f(o);
    }
  }
}

// Rows that fit in the registers of one thread block (up to 512 threads x 8 16-byte vectors):
// the row is read once, kept packed, and passes through max, exp / sum and the normalised store
// without touching memory again.  exp(v - m) is evaluated as 2^((v - m) * log2 e) on the
// special-function unit; masked (causal) positions produce exact zeros.
template <typename T, int VPT, bool kExact, bool kMasked>
__global__ void __launch_bounds__(512)
softmax_block_rows(const T* __restrict__ x, T* __restrict__ y, int cols, float scale, int causal, int64_t q_len) {
  using W = Words<T>;
  constexpr int EPW = W::EPW;
  constexpr int EPV = 4 * EPW;   // elements per 16-byte vector
  __shared__ float red[33];
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int nvec = cols / EPV;
  int valid = cols;
  if (kMasked && causal) {
    const int64_t v = (row % q_len) + (cols - q_len) + 1;
    valid = v > cols ? cols : (v < 0 ? 0 : static_cast<int>(v));
  }
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
  uint4 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) v[i] = __ldcs(xr + i * nthr + tid);
  const float c = scale * 1.4426950408889634f;   // scores are compared and exponentiated in log2 units
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) {
      const int e0 = (i * nthr + tid) * EPV;
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW];
        W::unpack(w[k], f);
#pragma unroll
        for (int e = 0; e < EPW; ++e)
          if (!kMasked || e0 + k * EPW + e < valid) m = fmaxf(m, f[e] * c);
      }
    }
  m = block_max(m, red);
  const float neg_m = m == -INFINITY ? 0.f : -m;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (kExact || i * nthr + tid < nvec) {
      const int e0 = (i * nthr + tid) * EPV;
      const uint32_t w[4] = {opaque(v[i].x), opaque(v[i].y), opaque(v[i].z), opaque(v[i].w)};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW];
        W::unpack(w[k], f);
#pragma unroll
        for (int e = 0; e < EPW; ++e)
          if (!kMasked || e0 + k * EPW + e < valid) s += exp2f_approx(fmaf(f[e], c, neg_m));
      }
    }
  s = block_sum(s, red);
  // the division by the row sum rides in the exponent: p / s = 2^(v - m - log2 s)
  const float shift = s > 0.f ? neg_m - log2f(s) : -INFINITY;
  uint4* yr = reinterpret_cast<uint4*>(y + row * cols);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = i * nthr + tid;
    if (kExact || vi < nvec) {
      const int e0 = vi * EPV;
      const uint32_t w[4] = {opaque(v[i].x), opaque(v[i].y), opaque(v[i].z), opaque(v[i].w)};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[EPW], r[EPW];
        W::unpack(w[k], f);
#pragma unroll
        for (int e = 0; e < EPW; ++e)
          r[e] = (!kMasked || e0 + k * EPW + e < valid) ? exp2f_approx(fmaf(f[e], c, shift)) : 0.f;
        o[k] = W::pack(r);
      }
      __stcs(yr + vi, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

template <typename T>
int launch_softmax(int64_t rows, int64_t cols, float scale, int causal, int64_t q_len,
                   const void* x, void* y, cudaStream_t stream) {
  constexpr int VW = Vec16<T>::N;
  const int64_t nvec = cols / VW;
  if (cols % VW == 0 && nvec <= 512 * 8 && aligned16(x) && aligned16(y) && rows <= 0x7fffffffll) {
    int threads = static_cast<int>((nvec + 7) / 8);
    threads = (threads + 31) / 32 * 32;
    const int vpt = static_cast<int>((nvec + threads - 1) / threads);
    const unsigned grid = static_cast<unsigned>(rows);
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    const int icols = static_cast<int>(cols);
    const bool exact = nvec == static_cast<int64_t>(threads) * (vpt <= 2 ? 2 : (vpt <= 4 ? 4 : 8));
#define KCG_SM_LAUNCH(V)                                                                                    \
  do {                                                                                                      \
    if (causal) {                                                                                           \
      if (exact) launch_overlapped(softmax_block_rows<T, V, true, true>, dim3(grid), dim3(threads), 0, stream, xp, yp, icols, scale, causal, q_len);   \
      else launch_overlapped(softmax_block_rows<T, V, false, true>, dim3(grid), dim3(threads), 0, stream, xp, yp, icols, scale, causal, q_len);        \
    } else {                                                                                                \
      if (exact) launch_overlapped(softmax_block_rows<T, V, true, false>, dim3(grid), dim3(threads), 0, stream, xp, yp, icols, scale, causal, q_len);  \
      else launch_overlapped(softmax_block_rows<T, V, false, false>, dim3(grid), dim3(threads), 0, stream, xp, yp, icols, scale, causal, q_len);       \
    }                                                                                                       \
  } while (0)
    if (vpt <= 2) KCG_SM_LAUNCH(2);
    else if (vpt <= 4) KCG_SM_LAUNCH(4);
    else KCG_SM_LAUNCH(8);
#undef KCG_SM_LAUNCH
    return check_launch("softmax_block_rows");
  }
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  softmax_rows<T><<<static_cast<int>(rows < cap ? rows : cap), 256, 0, stream>>>(
      static_cast<const T*>(x), static_cast<T*>(y), rows, cols, scale, causal, q_len);
  return check_launch("softmax_rows");
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_eltwise(int op, int dtype_in, int dtype_out, int64_t n, const void* x, void* y,
                           void* stream) {
  using namespace kcg;
  clear_error();
  if (n < 0) return fail(KCG_ERR_INVALID_ARG, "eltwise: negative element count");
  if (n == 0) return KCG_OK;
  if (!x || !y) return fail(KCG_ERR_INVALID_ARG, "eltwise: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (op != KCG_UNARY_CAST && dtype_in != dtype_out)
    return fail(KCG_ERR_INVALID_ARG, "eltwise: op %d needs dtype_out == dtype_in (got %d -> %d)", op,
                dtype_in, dtype_out);
  switch (op) {
    case KCG_UNARY_TANH: return dispatch_unary_same<OpTanh>(dtype_in, n, x, y, s);
    case KCG_UNARY_SQRT: return dispatch_unary_same<OpSqrt>(dtype_in, n, x, y, s);
    case KCG_UNARY_LOG: return dispatch_unary_same<OpLog>(dtype_in, n, x, y, s);
    case KCG_UNARY_RELU: return dispatch_unary_same<OpRelu>(dtype_in, n, x, y, s);
    case KCG_UNARY_GELU: return dispatch_unary_same<OpGelu>(dtype_in, n, x, y, s);
    case KCG_UNARY_CAST:
      switch (dtype_in) {
        case KCG_F32: return dispatch_cast_out<float>(dtype_out, n, x, y, s);
        case KCG_BF16: return dispatch_cast_out<__nv_bfloat16>(dtype_out, n, x, y, s);
        case KCG_F16: return dispatch_cast_out<__half>(dtype_out, n, x, y, s);
        case KCG_I32: return dispatch_cast_out<int32_t>(dtype_out, n, x, y, s);
        default: return fail(KCG_ERR_UNSUPPORTED, "eltwise Cast: source dtype %d has no kernel", dtype_in);
      }
    default: return fail(KCG_ERR_INVALID_ARG, "eltwise: unknown op %d", op);
  }
}

extern "C" int kcg_binary(int op, int dtype, int rank_a, const int64_t* shape_a, int rank_b,
                          const int64_t* shape_b, const void* a, const void* b, void* c,
                          void* stream) {
  using namespace kcg;
  clear_error();
  if (rank_a < 0 || rank_b < 0 || rank_a > KCG_MAX_RANK || rank_b > KCG_MAX_RANK)
    return fail(KCG_ERR_INVALID_ARG, "binary: rank out of range (%d, %d; max %d)", rank_a, rank_b, KCG_MAX_RANK);
  if ((rank_a && !shape_a) || (rank_b && !shape_b)) return fail(KCG_ERR_INVALID_ARG, "binary: null shape");
  const int rank = rank_a > rank_b ? rank_a : rank_b;
  // Trailing-aligned extents, innermost first; missing leading dims count as 1.
  int64_t ea[KCG_MAX_RANK], eb[KCG_MAX_RANK], eo[KCG_MAX_RANK];
  int64_t total = 1;
  bool same = true;
  for (int k = 0; k < rank; ++k) {
    ea[k] = k < rank_a ? shape_a[rank_a - 1 - k] : 1;
    eb[k] = k < rank_b ? shape_b[rank_b - 1 - k] : 1;
    if (ea[k] < 0 || eb[k] < 0) return fail(KCG_ERR_INVALID_ARG, "binary: negative extent");
    if (ea[k] != eb[k] && ea[k] != 1 && eb[k] != 1)
      return fail(KCG_ERR_INVALID_ARG, "binary: dim not equal (%lld vs %lld at trailing dim %d)",
                  static_cast<long long>(ea[k]), static_cast<long long>(eb[k]), k);
    eo[k] = ea[k] == 1 ? eb[k] : ea[k];
    if (ea[k] != eb[k]) same = false;
    total *= eo[k];
  }
  if (total == 0) return KCG_OK;
  if (!a || !b || !c) return fail(KCG_ERR_INVALID_ARG, "binary: null pointer");
  // Dense strides of each operand; 0 where it is broadcast.
  int64_t sa[KCG_MAX_RANK], sb[KCG_MAX_RANK];
  int64_t ra = 1, rb = 1;
  for (int k = 0; k < rank; ++k) {
    sa[k] = (ea[k] == 1 && eo[k] != 1) ? 0 : ra;
    sb[k] = (eb[k] == 1 && eo[k] != 1) ? 0 : rb;
    ra *= ea[k];
    rb *= eb[k];
  }
  // Collapse neighbours that both operands traverse contiguously (or both broadcast).
  BcastDims d;
  d.rank = 0;
  for (int k = 0; k < rank; ++k) {
    if (eo[k] == 1) continue;
    if (d.rank > 0) {
      const int p = d.rank - 1;
      if (sa[k] == d.stride_a[p] * d.extent[p] && sb[k] == d.stride_b[p] * d.extent[p]) {
        d.extent[p] *= eo[k];
        continue;
      }
    }
    d.extent[d.rank] = eo[k];
    d.stride_a[d.rank] = sa[k];
    d.stride_b[d.rank] = sb[k];
    ++d.rank;
  }
  if (d.rank == 0) {
    d.rank = 1;
    d.extent[0] = 1;
    d.stride_a[0] = 0;
    d.stride_b[0] = 0;
  }
  for (int k = d.rank; k < KCG_MAX_RANK; ++k) { d.extent[k] = 1; d.stride_a[k] = 0; d.stride_b[k] = 0; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (op) {
    case KCG_BINARY_ADD: return dispatch_binary_dtype<BAdd>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_MUL: return dispatch_binary_dtype<BMul>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_DIV: return dispatch_binary_dtype<BDiv>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_SUB: return dispatch_binary_dtype<BSub>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_POW: return dispatch_binary_dtype<BPow>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_EQUAL: return dispatch_binary_dtype<BEq>(dtype, d, same, total, a, b, c, s);
    case KCG_BINARY_GREATER: return dispatch_binary_dtype<BGt>(dtype, d, same, total, a, b, c, s);
    default: return fail(KCG_ERR_INVALID_ARG, "binary: unknown op %d", op);
  }
}

extern "C" int kcg_softmax(int dtype, int64_t rows, int64_t cols, float scale, int causal,
                           int64_t q_len, const void* x, void* y, void* stream) {
  using namespace kcg;
  clear_error();
  if (rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "softmax: negative size");
  if (rows == 0 || cols == 0) return KCG_OK;
  if (!x || !y) return fail(KCG_ERR_INVALID_ARG, "softmax: null pointer");
  if (causal && (q_len <= 0 || rows % q_len != 0))
    return fail(KCG_ERR_INVALID_ARG, "softmax: causal needs q_len > 0 dividing rows (rows=%lld q_len=%lld)",
                static_cast<long long>(rows), static_cast<long long>(q_len));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case KCG_F32: return launch_softmax<float>(rows, cols, scale, causal, q_len, x, y, s);
    case KCG_BF16: return launch_softmax<__nv_bfloat16>(rows, cols, scale, causal, q_len, x, y, s);
    case KCG_F16: return launch_softmax<__half>(rows, cols, scale, causal, q_len, x, y, s);
    default: return fail(KCG_ERR_UNSUPPORTED, "softmax: dtype %d has no kernel", dtype);
  }
}
