// Host side of the tensor-core GEMM (kernels and launch templates: gemm_kernels.cuh; their
// instantiations: gemm_inst_*.cu): tensor maps for the operands and the output, the choice of
// the tile shape, and the dispatch on element and output type.
#include "gemm_kernels.cuh"

#include <mutex>

namespace kcg {

int* device_status_word();  // runtime.cu: host-mapped word the kernels report faults into

namespace {

// ---- host side ----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

}  // namespace

// Encodes a rank-`rank` tensor map with 128-byte swizzle.  dims/strides are innermost
// first; strides (bytes) are given for dims 1..rank-1.
int encode_tmap_sw128(CUtensorMap* out, int dtype, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(KCG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMapDataType dt;
  switch (dtype) {
    case KCG_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case KCG_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case KCG_F8E4M3: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case KCG_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return fail(KCG_ERR_UNSUPPORTED, "tensor map: dtype %d", dtype);
  }
  cuuint64_t gd[5], gs[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(KCG_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu)",
                static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                static_cast<unsigned long long>(rank > 1 ? dims[1] : 1));
  return KCG_OK;
}

namespace {

// Per calling thread, so that two host threads (two generators, or a generator and a direct
// caller of the C ABI) never see each other's setting.
thread_local int g_pair_mode = -1;  // -1: pick_tiling(); 0: 128x256 single CTA; 1: CTA pairs when M > 128; 2: 128x128; 3: 128x64


// Chooses the CTA tile from a small cost model fitted to measurements on a B200 (microseconds):
// waves of tiles x time of one tile's main loop + a fixed cost per launch.  The unit is a 128x128
// block of output at the tensor pipe's full rate, 2.2 ns per element of K (four MMAs of
// 128x128x16 per 64 of K, 67.7 clocks each, at ~1.92 GHz).  The 256x256 pair tile and the 128x256
// tile are two such blocks per SM at that rate (the latter moves twice the operand bytes per SM
// and settles ~5 % lower under the power cap); the 128x128 and 128x64 tiles are bound by what one
// thread can issue, 377 and 365 clocks per k-block instead of 271 and 135, and pay only when the
// wider shapes would leave most SMs idle.  Fixed costs (launch, pipeline fill, the last tile's
// epilogue): 4.4 / 4.9 / 3.7 / 3.4 us measured for 128x256 / pair / 128x128 / 128x64.
Tiling pick_tiling(int64_t M, int64_t N, int64_t K, int64_t batch, int elem_bytes, int sms) {
  auto cdiv = [](int64_t a, int64_t b) { return (a + b - 1) / b; };
  // 8-bit inputs run at twice, tf32 at half the 16-bit rate
  const double unit = 2.2e-3 * static_cast<double>(K) * (elem_bytes == 1 ? 0.5 : (elem_bytes == 4 ? 2.0 : 1.0));
  const int64_t mt = cdiv(M, 128);
  const int64_t wide = mt * cdiv(N, 256) * batch, narrow = mt * cdiv(N, 128) * batch, slim = mt * cdiv(N, 64) * batch;
  const int64_t pairs = cdiv(M, 256) * cdiv(N, 256) * batch;
  const double c_wide = static_cast<double>(cdiv(wide, sms)) * 2 * 1.05 * unit + 4.4;
  const double c_narrow = static_cast<double>(cdiv(narrow, sms)) * 1.39 * unit + 3.7;
  const double c_slim = elem_bytes == 2 ? static_cast<double>(cdiv(slim, sms)) * 1.35 * unit + 3.4 : 1e30;
  const double c_pair = M >= 2 * BM ? static_cast<double>(cdiv(pairs, sms / 2)) * 2 * unit + 4.9 : 1e30;
  if (c_pair <= c_wide && c_pair <= c_narrow && c_pair <= c_slim) return kPair;
  if (c_wide <= c_narrow && c_wide <= c_slim) return kWide;
  return c_slim < c_narrow ? kSlim : kNarrow;
}

}  // namespace

// -1 (default): tile shape chosen by pick_tiling(); 0: 128x256 single-CTA tiles; 1: CTA pairs
// (cta_group::2, 256x256) whenever M > 128; 2: 128x128 single-CTA tiles; 3: 128x64 single-CTA tiles
// (16-bit inputs; 128x128 otherwise).
extern "C" __attribute__((visibility("default"))) void kcg_gemm_set_pair_mode(int mode) { g_pair_mode = mode; }

int gemm_tcgen05(int dtype_in, int dtype_out, int64_t M, int64_t N, int64_t K, int64_t batch, int trans_a,
                 int trans_b, const void* A, int64_t lda, int64_t stride_a, const void* B, int64_t ldb,
                 int64_t stride_b, void* C, int64_t ldc, int64_t stride_c, const float* scale_a,
                 const float* scale_b, const void* bias, int act, cudaStream_t stream, void* const* extra_c,
                 int n_extra, void* mc_c) {
  const int es = dtype_in == KCG_F8E4M3 ? 1 : (dtype_in == KCG_F32 ? 4 : 2);   // fp32 words are read as tf32
  if (!aligned16(A) || !aligned16(B))
    return fail(KCG_ERR_ALIGNMENT, "gemm: A and B must be 16-byte aligned for the tensor-core path");
  if ((lda * es) % 16 || (ldb * es) % 16 || (batch > 1 && ((stride_a * es) % 16 || (stride_b * es) % 16)))
    return fail(KCG_ERR_ALIGNMENT,
                "gemm: leading dimensions and batch strides must be multiples of 16 bytes (lda=%lld ldb=%lld)",
                static_cast<long long>(lda), static_cast<long long>(ldb));
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > INT32_MAX)
    return fail(KCG_ERR_UNSUPPORTED, "gemm: extents above 2^31-1 are not supported");

  const int BK = 128 / es;
  const uint32_t mn_box = 128 / es;
  Tiling tiling = g_pair_mode == 0 ? kWide
                  : g_pair_mode == 2 ? kNarrow
                  : g_pair_mode == 3 ? (es == 2 ? kSlim : kNarrow)
                  : g_pair_mode == 1 ? (M > BM ? kPair : kWide)
                                     : pick_tiling(M, N, K, batch, es, sm_count());
  if (n_extra > 0 || mc_c) {
    // only the CTA-pair kernel has the staged epilogue that writes whole 128-byte row segments
    if (n_extra > KCG_MAX_EXTRA_C) return fail(KCG_ERR_UNSUPPORTED, "gemm: at most %d extra outputs", KCG_MAX_EXTRA_C);
    if (M <= BM) return fail(KCG_ERR_UNSUPPORTED, "gemm: extra outputs need M > 128 (got %lld)", static_cast<long long>(M));
    tiling = kPair;
  }
  CUtensorMap tmA;
  BMaps bm;
  int a_blocked = 0, b_blocked = 0;
  {
    const uint64_t a_rows = trans_a ? K : M, a_cols = trans_a ? M : K;
    uint64_t dims[3] = {a_cols, a_rows, static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(lda) * es,
                           batch > 1 ? static_cast<uint64_t>(stride_a) * es : a_rows * static_cast<uint64_t>(lda) * es};
    uint32_t box[3];
    if (!trans_a) { box[0] = BK; box[1] = BM; } else { box[0] = mn_box; box[1] = BK; }
    box[2] = 1;
    a_blocked = trans_a && (M * es) % 128 == 0 && BM / mn_box > 1;
    int rc;
    if (a_blocked) {
      uint64_t d4[4] = {mn_box, a_rows, a_cols / mn_box, static_cast<uint64_t>(batch)};
      uint64_t s4[3] = {strides[0], 128, strides[1]};
      uint32_t b4[4] = {mn_box, static_cast<uint32_t>(BK), BM / mn_box, 1};
      rc = encode_tmap_sw128(&tmA, dtype_in, A, 4, d4, s4, b4);
    } else {
      rc = encode_tmap_sw128(&tmA, dtype_in, A, 3, dims, strides, box);
    }
    if (rc) return rc;
  }
  {
    const uint64_t b_rows = trans_b ? N : K, b_cols = trans_b ? K : N;
    uint64_t dims[3] = {b_cols, b_rows, static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(ldb) * es,
                           batch > 1 ? static_cast<uint64_t>(stride_b) * es : b_rows * static_cast<uint64_t>(ldb) * es};
    uint32_t box[3];
    if (trans_b) { box[0] = BK; box[1] = BN; } else { box[0] = mn_box; box[1] = BK; }
    box[2] = 1;
    b_blocked = !trans_b && (N * es) % 128 == 0;
    int rc;
    if (b_blocked) {
      uint64_t d4[4] = {mn_box, b_rows, b_cols / mn_box, static_cast<uint64_t>(batch)};
      uint64_t s4[3] = {strides[0], 128, strides[1]};
      uint32_t b4[4] = {mn_box, static_cast<uint32_t>(BK), BN / mn_box, 1};
      rc = encode_tmap_sw128(&bm.wide, dtype_in, B, 4, d4, s4, b4);
      if (rc) return rc;
      if (BN / 2 / mn_box > 1) {
        b4[2] = BN / 2 / mn_box;
        rc = encode_tmap_sw128(&bm.half, dtype_in, B, 4, d4, s4, b4);
      } else {
        rc = encode_tmap_sw128(&bm.half, dtype_in, B, 3, dims, strides, box);   // one block: the plain box
      }
      if (rc) return rc;
      rc = encode_tmap_sw128(&bm.quarter, dtype_in, B, 3, dims, strides, box);
      if (rc) return rc;
    } else {
    rc = encode_tmap_sw128(&bm.wide, dtype_in, B, 3, dims, strides, box);
    if (rc) return rc;
    // the CTA-pair kernel loads half of the B tile (128 of its 256 columns) per CTA; the 128- and
    // 64-wide single-CTA tiles use the same narrower boxes (an MN-major box is 128 bytes wide anyway)
    if (trans_b) box[1] = BN / 2;
    rc = encode_tmap_sw128(&bm.half, dtype_in, B, 3, dims, strides, box);
    if (rc) return rc;
    if (trans_b) box[1] = BN / 4;
    rc = encode_tmap_sw128(&bm.quarter, dtype_in, B, 3, dims, strides, box);
    if (rc) return rc;
    }
  }

  GemmParams p;
  p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.stride_c = stride_c;
  p.m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.n_tiles = static_cast<int>((N + BN - 1) / BN);
  p.total_tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * batch;
  p.k_blocks = static_cast<int>((K + BK - 1) / BK);
  p.scale_a = scale_a; p.scale_b = scale_b;
  p.bias = bias; p.act = act;
  p.status = device_status_word();
  if (!p.status) return fail(KCG_ERR_CUDA, "gemm: could not allocate the host-mapped status word");
  const size_t out_es = kcg_dtype_size(dtype_out);
  p.c_vec_ok = aligned16(C) && (ldc * out_es) % 16 == 0 && (stride_c * out_es) % 16 == 0;
  p.n_extra = n_extra;
  p.mc_c = mc_c;
  p.a_blocked = a_blocked; p.b_blocked = b_blocked;
  // C through TMA stores (boxes of 32 rows x 128 bytes) when its layout allows a tensor map
  CUtensorMap tmC;
  p.c_tma = 0;
  if (p.c_vec_ok && n_extra == 0 && !mc_c) {
    uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(ldc) * out_es,
                           batch > 1 ? static_cast<uint64_t>(stride_c) * out_es : static_cast<uint64_t>(M) * ldc * out_es};
    uint32_t box[3] = {static_cast<uint32_t>(128 / out_es), 32, 1};
    int rc = encode_tmap_sw128(&tmC, dtype_out, C, 3, dims, strides, box);
    if (rc) return rc;
    p.c_tma = 1;
  } else {
    tmC = tmA;   // never read
  }
  // 8, 32 and 64 were measured at 4096..16384: no better than 16 up to 8192^3; at 16384^3, where the
  // kernel is held back by DRAM traffic (22-34 GB per launch depending on the group), 32 reads the least
  p.group_m = static_cast<int64_t>(K) * es >= 32768 ? 2 * GROUP_M : GROUP_M;
  for (int i = 0; i < KCG_MAX_EXTRA_C; ++i) p.extra_c[i] = i < n_extra ? extra_c[i] : nullptr;
  if (n_extra > 0 || mc_c) {
    bool ok = p.c_vec_ok && (N * out_es) % 16 == 0 && aligned16(mc_c);
    for (int i = 0; i < n_extra; ++i) ok = ok && extra_c[i] != nullptr && aligned16(extra_c[i]);
    if (!ok)
      return fail(KCG_ERR_ALIGNMENT, "gemm: extra outputs need 16-byte aligned pointers, ldc and N (in bytes)");
  }

  const uint32_t a_mn = trans_a ? 1u : 0u, b_mn = trans_b ? 0u : 1u;
  if (dtype_in == KCG_F8E4M3) {
    const Idescs ids = {make_idesc(0, 0, a_mn, b_mn, BM, BN), make_idesc(0, 0, a_mn, b_mn, 2 * BM, BN),
                        make_idesc(0, 0, a_mn, b_mn, BM, 128), 0u};
    if (dtype_out == KCG_BF16)
      return gemm_launch_f8_bf16(trans_a, trans_b, tmA, bm, tmC, p, ids, tiling, stream);
    if (dtype_out == KCG_F32)
      return gemm_launch_f8_f32(trans_a, trans_b, tmA, bm, tmC, p, ids, tiling, stream);
    return fail(KCG_ERR_UNSUPPORTED, "gemm: float8_e4m3 inputs produce bfloat16 or float32 (got dtype %d)", dtype_out);
  }
  if (dtype_in == KCG_F32) {
    // tf32 operands (both K-major: the caller has laid them out that way), fp32 result
    if (trans_a || !trans_b || dtype_out != KCG_F32)
      return fail(KCG_ERR_UNSUPPORTED, "gemm: the tf32 path takes K-major operands and produces float32");
    const Idescs ids = {make_idesc(2, 2, 0, 0, BM, BN), make_idesc(2, 2, 0, 0, 2 * BM, BN), make_idesc(2, 2, 0, 0, BM, 128), 0u};
    return gemm_launch_tf32(0, 1, tmA, bm, tmC, p, ids, tiling, stream);
  }
  const uint32_t fmt = dtype_in == KCG_BF16 ? 1u : 0u;
  const Idescs ids = {make_idesc(fmt, fmt, a_mn, b_mn, BM, BN), make_idesc(fmt, fmt, a_mn, b_mn, 2 * BM, BN),
                      make_idesc(fmt, fmt, a_mn, b_mn, BM, 128), make_idesc(fmt, fmt, a_mn, b_mn, BM, 64)};
  if (dtype_out == KCG_F32) return gemm_launch_f16kind_f32(trans_a, trans_b, tmA, bm, tmC, p, ids, tiling, stream);
  if (dtype_in == KCG_BF16 && dtype_out == KCG_BF16)
    return gemm_launch_f16kind_bf16(trans_a, trans_b, tmA, bm, tmC, p, ids, tiling, stream);
  if (dtype_in == KCG_F16 && dtype_out == KCG_F16)
    return gemm_launch_f16kind_f16(trans_a, trans_b, tmA, bm, tmC, p, ids, tiling, stream);
  return fail(KCG_ERR_UNSUPPORTED, "gemm: dtype combination %d -> %d has no kernel", dtype_in, dtype_out);
}

}  // namespace kcg
