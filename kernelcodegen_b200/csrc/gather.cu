// Data-movement operators: Gather along one axis and Transpose of the two innermost dims.
//
// Gather follows the loop nest the reference builds for `Gather_{shape}_indices_{shape}_axis_{a}`
// (src/Frontend/Operators.cc:1253-1352): with the input viewed as [outer, axis_len, inner] and
// the indices flattened to n_idx values, out[o, i, r] = in[o, indices[i], r].  Both kernels are
// pure HBM traffic: 16-byte vectors wherever the inner extent allows it.
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace kcg {
int* device_status_word();  // runtime.cu
namespace {

template <typename I>
__device__ __forceinline__ int64_t checked_index(const I* __restrict__ indices, int64_t i, int64_t axis_len,
                                                 int* status) {
  int64_t k = static_cast<int64_t>(indices[i]);
  if (k < 0) k += axis_len;  // a negative index counts from the end
  if (k < 0 || k >= axis_len) {
    // record the fault and skip the access instead of reading out of bounds
    *status = KCG_ERR_INVALID_ARG;
    return -1;
  }
  return k;
}

// One thread per 16-byte vector of the output; `rv` vectors per gathered slice.
template <typename I>
__global__ void __launch_bounds__(256)
gather_vec(const uint4* __restrict__ in, const I* __restrict__ indices, uint4* __restrict__ out,
           int64_t total, int64_t n_idx, int64_t axis_len, int64_t rv, int* status) {
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = t % rv;
    const int64_t oi = t / rv;
    const int64_t i = oi % n_idx, o = oi / n_idx;
    const int64_t k = checked_index(indices, i, axis_len, status);
    uint4 val = make_uint4(0, 0, 0, 0);
    if (k >= 0) val = __ldg(in + (o * axis_len + k) * rv + v);
    __stcs(out + t, val);
  }
}

template <typename E, typename I>
__global__ void __launch_bounds__(256)
gather_scalar(const E* __restrict__ in, const I* __restrict__ indices, E* __restrict__ out,
              int64_t total, int64_t n_idx, int64_t axis_len, int64_t inner, int* status) {
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = t % inner;
    const int64_t oi = t / inner;
    const int64_t i = oi % n_idx, o = oi / n_idx;
    const int64_t k = checked_index(indices, i, axis_len, status);
    out[t] = k >= 0 ? in[(o * axis_len + k) * inner + r] : E(0);
  }
}

template <typename I>
int launch_gather(size_t esize, int64_t outer, int64_t axis_len, int64_t inner, int64_t n_idx, const void* in,
                  const I* indices, void* out, int* status, cudaStream_t stream) {
  const int64_t row_bytes = inner * static_cast<int64_t>(esize);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (row_bytes % 16 == 0 && aligned16(in) && aligned16(out)) {
    const int64_t rv = row_bytes / 16, total = outer * n_idx * rv;
    const int64_t blocks = std::min<int64_t>((total + 255) / 256, cap);
    gather_vec<I><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(in), indices, static_cast<uint4*>(out), total, n_idx, axis_len, rv, status);
    return check_launch("gather_vec");
  }
  const int64_t total = outer * n_idx * inner;
  const int64_t blocks = std::min<int64_t>((total + 255) / 256, cap);
#define KCG_GATHER(E)                                                                             \
  gather_scalar<E, I><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                         \
      static_cast<const E*>(in), indices, static_cast<E*>(out), total, n_idx, axis_len, inner, status)
  switch (esize) {
    case 1: KCG_GATHER(uint8_t); break;
    case 2: KCG_GATHER(uint16_t); break;
    case 4: KCG_GATHER(uint32_t); break;
    case 8: KCG_GATHER(uint64_t); break;
    default: return fail(KCG_ERR_UNSUPPORTED, "gather: element size %zu", esize);
  }
#undef KCG_GATHER
  return check_launch("gather_scalar");
}

// ---- transpose of the two innermost dims: out[b, j, i] = in[b, i, j] ---------------------
// A tile is TD x TD elements with TD = 32 * EPW, EPW elements per 32-bit word, so that a warp
// reads and writes 128 contiguous bytes whatever the element size.  The tile passes through
// shared memory as single elements (row pitch TD + EPW keeps the transposed reads spread over
// the banks for 4-byte elements and two-way at worst for smaller ones).
template <typename E>
__global__ void __launch_bounds__(256)
transpose_tiles(const E* __restrict__ in, E* __restrict__ out, int64_t R, int64_t C, int tiles_c, int tiles_r) {
  constexpr int EPW = sizeof(E) >= 4 ? 1 : 4 / sizeof(E);
  constexpr int TD = 32 * EPW;
  __shared__ E tile[TD][TD + EPW];
  const int64_t per_batch = static_cast<int64_t>(tiles_c) * tiles_r;
  const int64_t b = blockIdx.x / per_batch;
  const int tr = static_cast<int>((blockIdx.x % per_batch) / tiles_c);
  const int tc = static_cast<int>((blockIdx.x % per_batch) % tiles_c);
  const E* src = in + b * R * C;
  E* dst = out + b * R * C;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;  // 8 warps
  const int64_t r0 = static_cast<int64_t>(tr) * TD, c0 = static_cast<int64_t>(tc) * TD;
  const bool full = r0 + TD <= R && c0 + TD <= C;
  const bool word_in = full && (C % EPW == 0) && ((reinterpret_cast<uintptr_t>(in) & 3u) == 0);
  const bool word_out = full && (R % EPW == 0) && ((reinterpret_cast<uintptr_t>(out) & 3u) == 0);
  using Word = typename std::conditional<sizeof(E) >= 4, E, uint32_t>::type;
  // load: row r of the tile, word `lane`
  for (int r = w; r < TD; r += 8) {
    if (word_in) {
      const Word v = *reinterpret_cast<const Word*>(src + (r0 + r) * C + c0 + lane * EPW);
      const E* e = reinterpret_cast<const E*>(&v);
#pragma unroll
      for (int k = 0; k < EPW; ++k) tile[r][lane * EPW + k] = e[k];
    } else {
#pragma unroll
      for (int k = 0; k < EPW; ++k) {
        const int64_t rr = r0 + r, cc = c0 + lane * EPW + k;
        if (rr < R && cc < C) tile[r][lane * EPW + k] = src[rr * C + cc];
      }
    }
  }
  __syncthreads();
  // store: output row c (an input column), word `lane` = input rows lane*EPW ..
  for (int c = w; c < TD; c += 8) {
    if (word_out) {
      Word v;
      E* e = reinterpret_cast<E*>(&v);
#pragma unroll
      for (int k = 0; k < EPW; ++k) e[k] = tile[lane * EPW + k][c];
      *reinterpret_cast<Word*>(dst + (c0 + c) * R + r0 + lane * EPW) = v;
    } else {
#pragma unroll
      for (int k = 0; k < EPW; ++k) {
        const int64_t cc = c0 + c, rr = r0 + lane * EPW + k;
        if (cc < C && rr < R) dst[cc * R + rr] = tile[lane * EPW + k][c];
      }
    }
  }
}

// Wide-tile variant for 2- and 4-byte elements whose extents are tile multiples: a block moves
// 64 rows x 64 32-bit words (16 KB) with 16-byte global accesses, so that eight resident blocks
// keep well over 100 KB per SM in flight.  Shared memory holds words with an odd pitch; for
// 2-byte elements a word carries two horizontally adjacent elements and the store phase
// re-pairs the halves of two rows (a 2x2 transpose in registers).
template <int ES>
__global__ void __launch_bounds__(256)
transpose_wide(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int64_t R, int64_t C, int tiles_c,
               int tiles_r) {
  constexpr int EPW = 4 / ES;          // elements per word: 1 or 2
  constexpr int TR = 64, TW = 64;      // tile: 64 rows x 64 words (= 64 * EPW columns)
  constexpr int PITCH = TW + 1;
  __shared__ uint32_t tile[TR * PITCH];
  const int64_t per_batch = static_cast<int64_t>(tiles_c) * tiles_r;
  const int64_t b = blockIdx.x / per_batch;
  const int rem = static_cast<int>(blockIdx.x % per_batch);
  const int tr = rem / tiles_c, tc = rem % tiles_c;
  const int64_t in_pitch = C / EPW, out_pitch = R / EPW;   // row pitches in words
  const uint32_t* src = in + b * R * in_pitch + static_cast<int64_t>(tr) * TR * in_pitch + static_cast<int64_t>(tc) * TW;
  const int t = threadIdx.x;
  const int j = t & 15, rsub = t >> 4;   // 16 threads x 16 bytes span one 256-byte tile row
  uint4 v[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) v[p] = __ldcs(reinterpret_cast<const uint4*>(src + (p * 16 + rsub) * in_pitch) + j);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint32_t* row = tile + (p * 16 + rsub) * PITCH + 4 * j;
    row[0] = v[p].x; row[1] = v[p].y; row[2] = v[p].z; row[3] = v[p].w;
  }
  __syncthreads();
  if constexpr (EPW == 1) {
    // output row c (input column c) takes 64 words from input rows 0..63: 16 threads x 16 bytes
    uint32_t* dst = out + b * R * in_pitch + (static_cast<int64_t>(tc) * TW) * out_pitch + static_cast<int64_t>(tr) * TR;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int c = p * 16 + rsub;
      uint4 o;
      o.x = tile[(4 * j + 0) * PITCH + c]; o.y = tile[(4 * j + 1) * PITCH + c];
      o.z = tile[(4 * j + 2) * PITCH + c]; o.w = tile[(4 * j + 3) * PITCH + c];
      __stcs(reinterpret_cast<uint4*>(dst + c * out_pitch) + j, o);
    }
  } else {
    // 128 output rows (input columns) of 64 elements = 32 words each: 8 threads x 16 bytes per
    // row, 32 rows per pass.  Output word m of row c pairs in[2m][c] with in[2m+1][c].
    uint32_t* dst = out + b * R * in_pitch + (static_cast<int64_t>(tc) * TW * EPW) * out_pitch + static_cast<int64_t>(tr) * (TR / EPW);
    const int q = t & 7, csub = t >> 3;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int c = p * 32 + csub;           // element column inside the tile
      const int cw = c >> 1;
      const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;   // high halves or low halves of two words
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = tile[(8 * q + i) * PITCH + cw];
      uint4 o;
      o.x = __byte_perm(w[0], w[1], sel); o.y = __byte_perm(w[2], w[3], sel);
      o.z = __byte_perm(w[4], w[5], sel); o.w = __byte_perm(w[6], w[7], sel);
      __stcs(reinterpret_cast<uint4*>(dst + c * out_pitch) + q, o);
    }
  }
}

template <typename E>
int launch_transpose(int64_t batch, int64_t R, int64_t C, const void* in, void* out, cudaStream_t stream) {
  constexpr int EPW = sizeof(E) >= 4 ? 1 : 4 / sizeof(E);
  constexpr int TD = 32 * EPW;
  if constexpr (sizeof(E) == 2 || sizeof(E) == 4) {
    constexpr int ES = static_cast<int>(sizeof(E));
    constexpr int WCOLS = 64 * (4 / ES);   // tile width in elements
    if (R % 64 == 0 && C % WCOLS == 0 && aligned16(in) && aligned16(out)) {
      const int64_t wt_r = R / 64, wt_c = C / WCOLS, nblk = batch * wt_r * wt_c;
      if (nblk <= 0x7fffffffll) {
        transpose_wide<ES><<<static_cast<unsigned>(nblk), 256, 0, stream>>>(
            static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), R, C, static_cast<int>(wt_c), static_cast<int>(wt_r));
        return check_launch("transpose_wide");
      }
    }
  }
  const int64_t tiles_r = (R + TD - 1) / TD, tiles_c = (C + TD - 1) / TD;
  const int64_t blocks = batch * tiles_r * tiles_c;
  if (blocks > 0x7fffffffll || tiles_r > 0x7fffffffll || tiles_c > 0x7fffffffll)
    return fail(KCG_ERR_UNSUPPORTED, "transpose: more than 2^31 tiles");
  transpose_tiles<E><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const E*>(in), static_cast<E*>(out), R, C, static_cast<int>(tiles_c), static_cast<int>(tiles_r));
  return check_launch("transpose_tiles");
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_gather(int dtype, int index_dtype, int64_t outer, int64_t axis_len, int64_t inner,
                          int64_t n_idx, const void* input, const void* indices, void* output, void* stream) {
  using namespace kcg;
  clear_error();
  const size_t esize = kcg_dtype_size(dtype);
  if (esize == 0) return fail(KCG_ERR_INVALID_ARG, "gather: unknown dtype %d", dtype);
  if (index_dtype != KCG_I32 && index_dtype != KCG_I64)
    return fail(KCG_ERR_UNSUPPORTED, "gather: indices must be int32 or int64 (got dtype %d)", index_dtype);
  if (outer < 0 || axis_len < 0 || inner < 0 || n_idx < 0) return fail(KCG_ERR_INVALID_ARG, "gather: negative size");
  if (outer == 0 || inner == 0 || n_idx == 0) return KCG_OK;
  if (axis_len == 0) return fail(KCG_ERR_INVALID_ARG, "gather: the gathered axis is empty");
  if (!input || !indices || !output) return fail(KCG_ERR_INVALID_ARG, "gather: null pointer");
  int* status = device_status_word();
  if (!status) return fail(KCG_ERR_CUDA, "gather: could not allocate the host-mapped status word");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (index_dtype == KCG_I32)
    return launch_gather<int32_t>(esize, outer, axis_len, inner, n_idx, input, static_cast<const int32_t*>(indices),
                                  output, status, s);
  return launch_gather<int64_t>(esize, outer, axis_len, inner, n_idx, input, static_cast<const int64_t*>(indices),
                                output, status, s);
}

extern "C" int kcg_transpose(int dtype, int64_t batch, int64_t rows, int64_t cols, const void* input,
                             void* output, void* stream) {
  using namespace kcg;
  clear_error();
  const size_t esize = kcg_dtype_size(dtype);
  if (esize == 0) return fail(KCG_ERR_INVALID_ARG, "transpose: unknown dtype %d", dtype);
  if (batch < 0 || rows < 0 || cols < 0) return fail(KCG_ERR_INVALID_ARG, "transpose: negative size");
  if (batch == 0 || rows == 0 || cols == 0) return KCG_OK;
  if (!input || !output) return fail(KCG_ERR_INVALID_ARG, "transpose: null pointer");
  if (input == output) return fail(KCG_ERR_INVALID_ARG, "transpose: input and output must not alias");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (esize) {
    case 1: return launch_transpose<uint8_t>(batch, rows, cols, input, output, s);
    case 2: return launch_transpose<uint16_t>(batch, rows, cols, input, output, s);
    case 4: return launch_transpose<uint32_t>(batch, rows, cols, input, output, s);
    case 8: return launch_transpose<uint64_t>(batch, rows, cols, input, output, s);
    default: return fail(KCG_ERR_UNSUPPORTED, "transpose: element size %zu", esize);
  }
}
