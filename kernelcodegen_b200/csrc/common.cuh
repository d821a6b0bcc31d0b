// Shared host/device helpers for the sm_100a operator kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "kcg_kernels.h"

namespace kcg {

// Records a human-readable message for kcg_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

#define KCG_CUDA_OK(expr)                                                               \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::kcg::fail(KCG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                  \
                         cudaGetErrorString(_e), __FILE__, __LINE__);                   \
  } while (0)

// Returns KCG_OK if the launch that just happened was accepted by the runtime.
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(KCG_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return KCG_OK;
}

// ---- overlapped launches ------------------------------------------------------------
// A kernel launched with launch_overlapped() may become resident while the previous kernel in
// the stream is still draining (programmatic dependent launch): its CTAs take the SM slots that
// free up and block in grid_dependency_wait() until the previous grid has completed and its
// writes are visible.  The launch latency and the ramp-up of one kernel then hide under the tail
// of the one before, which is worth 1-2 us between two 25 us bandwidth kernels.
// Rule: every kernel launched this way calls grid_dependency_wait() in all threads before its
// first global access and calls grid_launch_dependents() once.  (A kernel that skipped the wait
// could finish before its predecessor and release its own successor too early.)
// Rule for kernels that allocate tensor memory: grid_launch_dependents() comes AFTER tcgen05.alloc
// has returned in the CTA.  A dependent grid starts only when every CTA of this grid has issued the
// trigger, so by then every resident CTA already holds its columns; if the trigger came first, a
// dependent CTA could become resident beside a CTA that has not allocated yet, take all 512
// columns and park in grid_dependency_wait(), and that CTA's tcgen05.alloc (a wait no time budget
// covers) would never return.
// KCG_OVERLAP_LAUNCH=0 in the environment launches the same kernels without the attribute, for A/B timing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool overlap_launch_enabled();
template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launch_enabled() ? 1 : 0;
  // an error is left for check_launch() (cudaGetLastError) to report
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

// ---- storage <-> fp32 conversion -------------------------------------------------
template <typename T> struct Conv;
template <> struct Conv<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Conv<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Conv<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Conv<int32_t> {
  static __device__ __forceinline__ float to_f(int32_t v) { return static_cast<float>(v); }
  static __device__ __forceinline__ int32_t from_f(float v) { return static_cast<int32_t>(v); }
};

// A 16-byte vector of T, loaded and stored with one 128-bit access.
template <typename T> struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld_vec(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
// Streaming variants: data that is touched once should not displace reusable lines.
template <typename T>
__device__ __forceinline__ Vec16<T> ld_vec_stream(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ void st_vec(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
template <typename T>
__device__ __forceinline__ void st_vec_stream(T* p, const Vec16<T>& r) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
}

// 32-byte (256-bit) streaming accesses: one instruction per thread where an operand is twice as
// wide as the other (Cast between 16- and 32-bit types).  The address must be 32-byte aligned.
__device__ __forceinline__ void ld_256(const void* p, uint4& lo, uint4& hi) {
  asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
               : "l"(p));
}
__device__ __forceinline__ void st_256(void* p, const uint4& lo, const uint4& hi) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(lo.x), "r"(lo.y), "r"(lo.z),
               "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
               : "memory");
}

// One 16-byte store to a multicast address: NVSwitch writes it into the buffer of every GPU bound
// to the multicast object (the issuing GPU's own included), so a gather that needs the same bytes on
// N GPUs sends them over this GPU's links once instead of N - 1 times.  A data move: the four words
// pass through float registers untouched.
__device__ __forceinline__ void multimem_st16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the whole thread block; every thread receives the result.
// `scratch` holds at least 33 floats of shared memory.  Safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (nwarps == 1) return v;
  __syncthreads();  // protect scratch from the previous call's readers
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (nwarps == 1) return v;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  return warp_max(t);
}


// GELU in the reference's tanh form, with its literal constants and its operation order
// (src/Frontend/Operators.cc:981-995): 0.5x * (tanh(0.797884 * (0.044715 * (x * (x*x)) + x)) + 1).
// Every step is an explicitly rounded multiply or add, so no call site can be contracted into
// FMAs differently from another: the stand-alone kernel and the fused kernels agree bit for bit.
// kFast uses the hardware tanh approximation (error below the rounding of a 16-bit result).
template <bool kFast>
__device__ __forceinline__ float gelu_tanh(float v) {
  const float t1 = __fmul_rn(v, 0.5f);
  const float t3 = __fmul_rn(v, __fmul_rn(v, v));
  const float t5 = __fadd_rn(__fmul_rn(0.044715f, t3), v);
  const float t6 = __fmul_rn(0.797884f, t5);
  float t7;
  if constexpr (kFast) {
    asm("tanh.approx.f32 %0, %1;" : "=f"(t7) : "f"(t6));
  } else {
    t7 = tanhf(t6);
  }
  return __fmul_rn(t1, __fadd_rn(t7, 1.0f));
}

// The same function for two values at once with packed fp32x2 instructions (each lane of
// mul / add .rn.f32x2 rounds exactly like the scalar instruction, and the operation sequence is
// the scalar one, so the results are the bits gelu_tanh() gives); 8 packed instructions and two
// tanh instead of 16 + 2.
template <bool kFast>
__device__ __forceinline__ void gelu_tanh_pair(float& a, float& b) {
  if constexpr (!kFast) {
    a = gelu_tanh<false>(a);
    b = gelu_tanh<false>(b);
  } else {
    uint64_t v, half2v, c1, c0, one, t1, vv, t3, m, t5, t6;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(a), "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(half2v) : "f"(0.5f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "f"(0.044715f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "f"(0.797884f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(one) : "f"(1.0f));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t1) : "l"(v), "l"(half2v));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(vv) : "l"(v), "l"(v));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t3) : "l"(v), "l"(vv));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(m) : "l"(c1), "l"(t3));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(t5) : "l"(m), "l"(v));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t6) : "l"(c0), "l"(t5));
    float x0, x1, y0, y1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(t6));
    asm("tanh.approx.f32 %0, %1;" : "=f"(y0) : "f"(x0));
    asm("tanh.approx.f32 %0, %1;" : "=f"(y1) : "f"(x1));
    uint64_t t7, s, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(t7) : "f"(y0), "f"(y1));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(s) : "l"(t7), "l"(one));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(t1), "l"(s));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r));
  }
}

// 2^x on the special-function unit (relative error about 2^-22, denormal results flushed).
__device__ __forceinline__ float exp2f_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Two fp32 values in one 64-bit register for the packed .f32x2 instructions of sm_100 (each lane
// rounds like the scalar instruction).
__device__ __forceinline__ uint64_t pk_make(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void pk_split(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t pk_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t pk_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// Row kernels (LayerNorm, softmax) keep a row in registers as raw 32-bit words (two 16-bit
// elements or one fp32 per word) and unpack it once per pass over the row.  Keeping the packed
// form (a bf16 row of 4096 is 64 registers per lane at one warp per row) is what lets enough
// warps be resident to cover HBM latency; `opaque` stops the compiler from keeping an unpacked
// fp32 copy alive across the passes instead.
template <typename T> struct Words;
template <> struct Words<float> {
  static constexpr int EPW = 1;
  static __device__ __forceinline__ void unpack(uint32_t w, float (&f)[1]) { f[0] = __uint_as_float(w); }
  static __device__ __forceinline__ uint32_t pack(const float (&f)[1]) { return __float_as_uint(f[0]); }
};
template <> struct Words<__nv_bfloat16> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void unpack(uint32_t w, float (&f)[2]) {
    f[0] = __uint_as_float(w << 16);
    f[1] = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack(const float (&f)[2]) {
    __nv_bfloat162 v = __floats2bfloat162_rn(f[0], f[1]);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Words<__half> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void unpack(uint32_t w, float (&f)[2]) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w));
    f[0] = v.x;
    f[1] = v.y;
  }
  static __device__ __forceinline__ uint32_t pack(const float (&f)[2]) {
    __half2 v = __floats2half2_rn(f[0], f[1]);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
__device__ __forceinline__ uint32_t opaque(uint32_t w) {
  asm volatile("" : "+r"(w));
  return w;
}

// Fused GEMM epilogue: out = act(alpha * acc + bias), rounded to TOut after each step where the
// unfused chain (Matmul -> Binary Add -> ElementWise) would have stored the intermediate, so
// the fused result is bit-identical to the chain.  act: 0 none, 1 Relu, 2 Gelu (tanh form with
// the reference's constants, evaluated like the stand-alone elementwise kernel).
template <typename TOut>
__device__ __forceinline__ TOut gemm_epilogue_value(float acc, float alpha, const TOut* __restrict__ bias,
                                                    int64_t col, int act) {
  TOut v = Conv<TOut>::from_f(alpha * acc);
  if (bias) v = Conv<TOut>::from_f(Conv<TOut>::to_f(v) + Conv<TOut>::to_f(bias[col]));
  if (act == 1) {
    v = Conv<TOut>::from_f(fmaxf(0.f, Conv<TOut>::to_f(v)));
  } else if (act == 2) {
    v = Conv<TOut>::from_f(gelu_tanh<(sizeof(TOut) < 4)>(Conv<TOut>::to_f(v)));
  }
  return v;
}

}  // namespace kcg
