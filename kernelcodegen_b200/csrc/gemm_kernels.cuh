// Tensor-core GEMM for sm_100a: C = alpha * op(A) * op(B), 16-bit and FP8 inputs, fp32
// accumulation in tensor memory.
//
// This replaces the kernel the reference emits for Matmul / BatchMatmul
// (src/Optimizer/Optimizer.cc:406-570, :3290-3445): a 128x128x8 CUDA-core tile with a
// register/shared double buffer.  The Blackwell design keeps the same roles — stage
// operand tiles in shared memory, accumulate a C tile on chip, write it once — but maps
// them to the hardware units that exist for it:
//   warp 0      TMA producer (one thread): cp.async.bulk.tensor loads of 128-byte-swizzled A
//               and B tiles into a ring, completion counted on mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256/128/64, K=32 bytes) from
//               shared-memory descriptors into one of two fp32 accumulators in tensor memory,
//               and releases ring entries with tcgen05.commit;
//   warps 2-9   epilogue: tcgen05.ld the finished accumulator (two warps per TMEM lane quarter,
//               each half of the columns), scale, convert and store, while the MMA warp already
//               fills the other accumulator with the next tile.
// CTAs are persistent (one per SM) and walk the tile list in an M-grouped order so that
// the tiles in flight share A row-blocks and B column-blocks in L2 (the reference's
// unused GROUP_SIZE_M, include/KernelCodeGen.h:36).
//
// Both operand layouts of the reference API are handled without a transpose pass: a
// row-major [M,K] A or [N,K] B tile is "K-major" for the MMA, a row-major [K,M] A or
// [K,N] B tile (the plain Matmul's B) is "MN-major"; only the TMA box shape and two
// descriptor fields differ.
//
// This header holds the kernels and their launch templates; gemm_tcgen05.cu holds the host side
// (tensor maps, tile choice) and gemm_inst_*.cu instantiate the kernels, one unit per operand /
// output type so that they compile side by side.
#pragma once
#include "common.cuh"
#include "tcgen05.cuh"

namespace kcg {

#define KCG_MAX_EXTRA_C 7

// ---- types shared by the host side and the instantiation units
struct GemmParams {
  void* C;
  int64_t M, N, K;
  int64_t ldc, stride_c;
  int m_tiles, n_tiles;
  int64_t total_tiles;
  int k_blocks;
  const float* scale_a;
  const float* scale_b;
  int* status;
  int c_vec_ok;
  const void* bias;  // N values of the output dtype, or null
  int act;           // 0 none, 1 Relu, 2 Gelu
  // Further copies of C (same ldc / stride_c), typically this rank's block inside the gather
  // buffers of peer GPUs: the CTA-pair kernel's epilogue stores every tile to each of them.
  void* extra_c[KCG_MAX_EXTRA_C];
  int n_extra;
  // Or: the same block of C inside a multicast mapping of every rank's gather buffer; each tile is
  // then stored once, to this address, instead of to C and every extra_c.
  void* mc_c;
  int group_m;   // row tiles (of 128) per group of the tile order
  // An MN-major operand whose rows are whole 128-byte blocks is described by a rank-4 map
  // {128 bytes, K, blocks, batch}: one TMA copy then brings all column blocks of a tile (the
  // copy engine, not the issuing thread, pays a fixed price per copy: an MN-major B tile of 256
  // columns in four copies held the 128x256 kernel at 650-700 clocks per k-block instead of 545).
  int a_blocked, b_blocked;
  int c_tma;     // C is written with TMA stores from a staged tile (needs c_vec_ok; see epilogue_rows_tma)
};

enum Tiling { kWide = 0, kPair = 1, kNarrow = 2, kSlim = 3 };
struct Idescs { uint32_t wide, pair, narrow, slim; };
struct BMaps { CUtensorMap wide, half, quarter; };   // B boxes of 256, 128 and 64 columns of the tile

// One entry per instantiation unit (gemm_inst_*.cu): element kind x output type, all four operand
// layouts and all four tile shapes inside.
#define KCG_GEMM_LAUNCH_ARGS                                                                             \
  int trans_a, int trans_b, const CUtensorMap &tmA, const BMaps &bm, const CUtensorMap &tmC,            \
      const GemmParams &p, const Idescs &idescs, Tiling tiling, cudaStream_t s
int gemm_launch_f16kind_bf16(KCG_GEMM_LAUNCH_ARGS);   // bf16 in, bf16 out
int gemm_launch_f16kind_f16(KCG_GEMM_LAUNCH_ARGS);    // fp16 in, fp16 out
int gemm_launch_f16kind_f32(KCG_GEMM_LAUNCH_ARGS);    // bf16 / fp16 in, fp32 out
int gemm_launch_f8_bf16(KCG_GEMM_LAUNCH_ARGS);        // e4m3 in, bf16 out
int gemm_launch_f8_f32(KCG_GEMM_LAUNCH_ARGS);         // e4m3 in, fp32 out
int gemm_launch_tf32(KCG_GEMM_LAUNCH_ARGS);           // tf32 (K-major operands), fp32 out

namespace {
using namespace sm100;


constexpr int BM = 128, BN = 256;
constexpr int A_BYTES = BM * 128;
constexpr int EPI_WARPS = 8;                     // two per tensor-memory lane quarter
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUP_M = 16;
constexpr int EPI_STAGE_BYTES = 32 * 128;            // per epilogue warp: 32 rows x 128 bytes of output on their way out
constexpr int RING_BYTES = 4 * (A_BYTES + BN * 128);  // = 6 x 32 KB (128-wide tile) = 8 x 24 KB (64-wide tile)
constexpr int SMEM_BYTES = RING_BYTES + EPI_WARPS * EPI_STAGE_BYTES + 1024 + 256;


__device__ __forceinline__ void tile_coords(int64_t tile, const GemmParams& p, int& b, int& mt, int& nt) {
  const int64_t per_batch = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  b = static_cast<int>(tile / per_batch);
  const int r = static_cast<int>(tile % per_batch);
  const int group_span = p.group_m * p.n_tiles;
  const int group = r / group_span;
  const int first_m = group * p.group_m;
  const int gsize = min(p.m_tiles - first_m, p.group_m);
  const int in_group = r % group_span;
  mt = first_m + in_group % gsize;
  nt = in_group / gsize;
}

// 16 bytes of output from VW consecutive accumulators scaled by alpha (no bias, no activation):
// the same fmul + round-to-nearest as gemm_epilogue_value, with two results per conversion.
template <typename TOut> __device__ __forceinline__ uint4 scale_pack16(const uint32_t* r, float alpha);
template <> __device__ __forceinline__ uint4 scale_pack16<float>(const uint32_t* r, float alpha) {
  return make_uint4(__float_as_uint(alpha * __uint_as_float(r[0])), __float_as_uint(alpha * __uint_as_float(r[1])),
                    __float_as_uint(alpha * __uint_as_float(r[2])), __float_as_uint(alpha * __uint_as_float(r[3])));
}
template <> __device__ __forceinline__ uint4 scale_pack16<__nv_bfloat16>(const uint32_t* r, float alpha) {
  uint4 o;
  __nv_bfloat162 v;
  v = __floats2bfloat162_rn(alpha * __uint_as_float(r[0]), alpha * __uint_as_float(r[1])); o.x = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2bfloat162_rn(alpha * __uint_as_float(r[2]), alpha * __uint_as_float(r[3])); o.y = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2bfloat162_rn(alpha * __uint_as_float(r[4]), alpha * __uint_as_float(r[5])); o.z = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2bfloat162_rn(alpha * __uint_as_float(r[6]), alpha * __uint_as_float(r[7])); o.w = *reinterpret_cast<uint32_t*>(&v);
  return o;
}
template <> __device__ __forceinline__ uint4 scale_pack16<__half>(const uint32_t* r, float alpha) {
  uint4 o;
  __half2 v;
  v = __floats2half2_rn(alpha * __uint_as_float(r[0]), alpha * __uint_as_float(r[1])); o.x = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2half2_rn(alpha * __uint_as_float(r[2]), alpha * __uint_as_float(r[3])); o.y = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2half2_rn(alpha * __uint_as_float(r[4]), alpha * __uint_as_float(r[5])); o.z = *reinterpret_cast<uint32_t*>(&v);
  v = __floats2half2_rn(alpha * __uint_as_float(r[6]), alpha * __uint_as_float(r[7])); o.w = *reinterpret_cast<uint32_t*>(&v);
  return o;
}

// Epilogue of one thread for its row of a finished accumulator (kTileN columns starting at
// col0): tensor memory is read 64 columns per round trip; full, aligned blocks without bias or
// activation take the packed path above, everything else goes element by element.
//
// kChunk columns travel per round trip (64, or 32 for the 64-wide tile); a thread takes the chunks
// first, first + step, ... so that two warps on the same lane quarter can share a row.
template <typename TOut, int kTileN, int kChunk = 64>
__device__ __forceinline__ void epilogue_row(uint32_t t_base, TOut* crow, bool row_ok, int64_t col0,
                                             const GemmParams& p, float alpha, const TOut* bias,
                                             int first = 0, int step = 1) {
  constexpr int VW = Vec16<TOut>::N;
  const bool plain = bias == nullptr && p.act == 0 && p.c_vec_ok != 0;
#pragma unroll 1
  for (int c = first; c < kTileN / kChunk; c += step) {
    uint32_t r[kChunk];
    if constexpr (kChunk == 64) tmem_ld64(t_base + c * kChunk, r); else tmem_ld32(t_base + c * kChunk, r);
    tmem_wait_ld();
    if (!row_ok) continue;
    const int64_t cbase = col0 + c * kChunk;
    if (plain && cbase + kChunk <= p.N) {
#pragma unroll
      for (int g = 0; g < kChunk / VW; ++g)
        *reinterpret_cast<uint4*>(crow + cbase + g * VW) = scale_pack16<TOut>(&r[g * VW], alpha);
    } else {
#pragma unroll
      for (int g = 0; g < kChunk / VW; ++g) {
        const int64_t col = cbase + g * VW;
        if (p.c_vec_ok && col + VW <= p.N) {
          Vec16<TOut> o;
#pragma unroll
          for (int j = 0; j < VW; ++j) o.v[j] = gemm_epilogue_value<TOut>(__uint_as_float(r[g * VW + j]), alpha, bias, col + j, p.act);
          st_vec(crow + col, o);
        } else {
#pragma unroll
          for (int j = 0; j < VW; ++j)
            if (col + j < p.N) crow[col + j] = gemm_epilogue_value<TOut>(__uint_as_float(r[g * VW + j]), alpha, bias, col + j, p.act);
        }
      }
    }
  }
}

// The same rows written through shared memory and TMA.  One thread per accumulator row is how
// tensor memory hands the data out, but stored that way every warp instruction touches 32
// different 128-byte lines with 16 bytes each — a 128x256 tile of 16-bit outputs is 4096 such
// sector writes and took about 2 us, all of it exposed when a CTA has a single tile.  Here a warp
// packs 128 bytes per row into a swizzled 4 KB staging tile of its own and one lane hands the
// 32-row box to the copy engine, which writes whole lines and clips at M and N.
// `spare`, when not null, is shared memory nobody else uses any more (the operand ring after the
// CTA's last tile) with room for every round of this warp: the rounds then need not wait for
// one another's staging tile, which matters when nothing else hides the epilogue.
template <typename TOut, int kTileN>
__device__ __forceinline__ void epilogue_rows_tma(uint32_t t_base, uint8_t* stg, const CUtensorMap* tmC, int row0, int col0,
                                                  int batch, const GemmParams& p, float alpha, const TOut* bias,
                                                  int first, int step, int lane, uint8_t* spare = nullptr) {
  constexpr int VW = Vec16<TOut>::N;
  constexpr int RC = 128 / static_cast<int>(sizeof(TOut));   // columns per round: 128 bytes of output per row
  const bool plain = bias == nullptr && p.act == 0;
  bool pending = false;
#pragma unroll 1
  for (int c = first; c < kTileN / RC; c += step) {
    uint32_t r[RC];
    if constexpr (RC == 64) tmem_ld64(t_base + c * RC, r); else tmem_ld32(t_base + c * RC, r);
    tmem_wait_ld();
    const int cbase = col0 + c * RC;
    if (cbase >= p.N || row0 >= p.M) continue;   // nothing of this box lies inside C
    if (spare != nullptr) {
      stg = spare;
      spare += EPI_STAGE_BYTES;
    } else if (pending) {   // the copy engine has read the previous round out of the staging tile
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      uint4 v;
      if (plain) {
        v = scale_pack16<TOut>(&r[g * VW], alpha);
      } else {
        Vec16<TOut> o;
        const int64_t col = cbase + g * VW;
#pragma unroll
        for (int j = 0; j < VW; ++j)
          o.v[j] = col + j < p.N ? gemm_epilogue_value<TOut>(__uint_as_float(r[g * VW + j]), alpha, bias, col + j, p.act)
                                 : TOut(0.f);
        v = *reinterpret_cast<const uint4*>(&o);
      }
      *reinterpret_cast<uint4*>(stg + lane * 128 + ((g ^ (lane & 7)) << 4)) = v;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(tmC, stg, cbase, row0, batch);
      tma_store_commit();
    }
    pending = true;
  }
  // The staging tile must have been read before the warp reuses it or the CTA exits and its
  // shared memory goes away; that the bytes have reached global memory is the kernel boundary's
  // business, as for any other store.
  if (pending && lane == 0) tma_store_wait_read<0>();
  __syncwarp();
}

// kBN: width of the CTA tile, 256 (4-stage ring of 48 KB), 128 (6 stages of 32 KB) or 64 (8 stages
// of 24 KB).  The narrower tiles cost more shared-memory and L2 traffic per flop but quantise
// better: they are chosen when the problem has too few wide tiles to fill the SMs (see
// pick_tiling()).  Eight epilogue warps, two per tensor-memory lane quarter, split a tile's columns:
// small problems run one tile per CTA, so nothing hides the epilogue and its latency counts in full.
template <Kind kKind, int kElemBytes, bool kAMn, bool kBMn, typename TOut, int kBN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p, const uint32_t idesc) {
  constexpr int BN = kBN;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = kBN == 256 ? 4 : (kBN == 128 ? 6 : 8);
  // Ring entries ("units") of kSub stages share one pair of barriers: the MMA thread's cost per
  // k-block, not the tensor pipe, bounds the narrow tiles, and a commit per 64 of K is a large
  // part of it: two k-blocks per unit for the 128-wide tile (three units), four for the 64-wide
  // one (two units, one in use and one loading).  The wide tile is pipe-bound and keeps the finer
  // ring.
  constexpr int kSub = kBN == 256 ? 1 : (kBN == 128 ? 2 : 4);
  constexpr int UNITS = STAGES / kSub;
  constexpr int BK = 128 / kElemBytes;             // elements per k-block (128 bytes of K)
  constexpr int UMMA_K = 32 / kElemBytes;          // elements per MMA (32 bytes of K)
  constexpr int MN_BOX = 128 / kElemBytes;         // inner extent of an MN-major TMA box
  constexpr int MN_BOX_BYTES = BK * 128;           // one MN-major box: BK k-rows of 128 bytes
  constexpr int MN_KSTEP = UMMA_K * 128;           // bytes between MMA k-steps, MN-major

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  static_assert(STAGES * STAGE_BYTES == RING_BYTES, "every tile width uses the whole ring");
  uint8_t* epi_stage = smem + RING_BYTES;    // [EPI_WARPS] x 4 KB, 1024-byte aligned like the ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_WARPS * EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint64_t* drain_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.c_tma) prefetch_tmap(&tmC);
    for (int s = 0; s < UNITS; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The next kernel's prologue may overlap this kernel from here on (see launch_overlapped), and
  // only from here: this CTA holds its tensor memory now (the rule in common.cuh).
  grid_launch_dependents();
  // Barriers, tensor memory and descriptors are set up; operands and the output may be touched
  // only when the kernel before this one in the stream has finished.
  grid_dependency_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0, s = 0, ph = 0;   // it: ring units filled so far; s, ph: unit and its phase
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        int b, mt, nt;
        tile_coords(tile, p, b, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < p.k_blocks; kb += kSub, ++it, ph ^= (s + 1 == UNITS), s = (s + 1 == UNITS ? 0 : s + 1)) {
          // the first pass over the ring finds every unit free without asking
          if (it >= UNITS && !mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          const int nsub = min(kSub, p.k_blocks - kb);
          mbar_expect_tx(&full_bar[s], nsub * STAGE_BYTES);
#pragma unroll
          for (int u = 0; u < kSub; ++u) {
            if (u >= nsub) break;
            uint8_t* a_dst = smem + (s * kSub + u) * STAGE_BYTES;
            uint8_t* b_dst = a_dst + A_BYTES;
            const int k0 = (kb + u) * BK;
            if constexpr (!kAMn) {
              tma_load_3d(a_dst, &tmA, &full_bar[s], k0, m0, b);
            } else if (p.a_blocked && A_BYTES / MN_BOX_BYTES > 1) {
              tma_load_4d(a_dst, &tmA, &full_bar[s], 0, k0, m0 / MN_BOX, b);   // all 128-byte column blocks in one copy
            } else {
#pragma unroll
              for (int j = 0; j < A_BYTES / MN_BOX_BYTES; ++j)
                tma_load_3d(a_dst + j * MN_BOX_BYTES, &tmA, &full_bar[s], m0 + j * MN_BOX, k0, b);
            }
            if constexpr (!kBMn) {
              tma_load_3d(b_dst, &tmB, &full_bar[s], k0, n0, b);
            } else if (p.b_blocked && B_BYTES / MN_BOX_BYTES > 1) {
              tma_load_4d(b_dst, &tmB, &full_bar[s], 0, k0, n0 / MN_BOX, b);
            } else {
#pragma unroll
              for (int j = 0; j < B_BYTES / MN_BOX_BYTES; ++j)
                tma_load_3d(b_dst + j * MN_BOX_BYTES, &tmB, &full_bar[s], n0 + j * MN_BOX, k0, b);
            }
          }
        }
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        // Let the copies that were already issued land before the CTA goes away.
        int zero = 0;
        const uint32_t first = it > UNITS ? it - UNITS : 0;
        for (uint32_t j = first; j < it; ++j)
          mbar_wait(&full_bar[j % UNITS], (j / UNITS) & 1u, &zero, 2000000ull);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // A single thread runs the loop.  An MMA is accepted only when the tensor pipe has room,
    // so every instruction between two MMAs competes with the pipe's run time: the descriptors
    // of a stage are derived from one precomputed base by integer adds, and no other lane
    // takes part (no reconvergence after the barrier waits).
    if (lane == 0) {
      uint32_t tile_iter = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      // Descriptors of k-step 0 in stage 0; later k-steps / stages differ only in the address
      // field (bits [0,14), in 16-byte units), which cannot carry into the next field here.
      const uint64_t adesc0 = kAMn ? make_smem_desc(smem_base, MN_BOX_BYTES, 1024) : make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = kBMn ? make_smem_desc(smem_base + A_BYTES, MN_BOX_BYTES, 1024)
                                   : make_smem_desc(smem_base + A_BYTES, 16, 1024);
      constexpr uint32_t kStageStep = STAGE_BYTES >> 4;
      constexpr uint32_t kAStep = (kAMn ? MN_KSTEP : 32) >> 4, kBStep = (kBMn ? MN_KSTEP : 32) >> 4;
      static_assert(BK / UMMA_K == 4, "mma_kblock issues four k-steps");
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      // s / ph walk the ring of units; `ready` says that the unit about to be used was already
      // seen full by the test that rode along with the previous unit's last MMAs.
      uint32_t s = 0, ph = 0;
      bool ready = false;
      for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; kb += kSub) {
          if (!ready && !mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t s1 = s + 1 == UNITS ? 0u : s + 1, ph1 = s + 1 == UNITS ? ph ^ 1u : ph;
          uint32_t slot = s * kSub;
          if constexpr (kSub > 1) {
            // all but the last k-block of the unit: MMAs only
            for (int u = 0; u + 1 < kSub && kb + u + 1 < p.k_blocks; ++u, ++slot) {
              const uint64_t adesc = adesc0 + slot * kStageStep, bdesc = bdesc0 + slot * kStageStep;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_ss<kKind>(d_tmem, adesc + k * kAStep, bdesc + k * kBStep, idesc, (kb | u | k) != 0 ? 1u : 0u);
            }
          }
          ready = mma_kblock<kKind, false>(d_tmem, adesc0 + slot * kStageStep, bdesc0 + slot * kStageStep, kAStep, kBStep,
                                           idesc, (kb != 0 || slot != s * kSub) ? 1u : 0u, empty0 + s * 8, 0,
                                           full0 + s1 * 8, ph1);
          s = s1; ph = ph1;
        }
        if (ok) mma_commit(&tfull_bar[acc]);
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit(drain_bar);
        mbar_wait(drain_bar, 0, &zero, 20000000ull);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    float alpha = 1.f;
    if (p.scale_a) alpha *= *p.scale_a;
    if (p.scale_b) alpha *= *p.scale_b;
    const TOut* bias = static_cast<const TOut*>(p.bias);
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++tile_iter) {
      int b, mt, nt;
      tile_coords(tile, p, b, mt, nt);
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = static_cast<int64_t>(mt) * BM + quarter * 32 + lane;
      const int64_t col0 = static_cast<int64_t>(nt) * BN;
      TOut* crow = static_cast<TOut*>(p.C) + b * p.stride_c + row * p.ldc;
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      // (the 64-wide tile has so little to store per warp that the staging round trip costs more
      // than the scattered stores: 6.15 against 6.45 us at 1024^3)
      if (p.c_tma && BN >= 128)
        epilogue_rows_tma<TOut, BN>(t_base, epi_stage + (warp - 2) * EPI_STAGE_BYTES, &tmC, mt * BM + quarter * 32,
                                    static_cast<int>(col0), b, p, alpha, bias, col_half, EPI_WARPS / 4, lane,
                                    // after the CTA's last tile the operand ring is idle: 16 KB of it per warp
                                    tile + gridDim.x >= p.total_tiles ? smem + (warp - 2) * 16384 : nullptr);
      else
        epilogue_row<TOut, BN, (BN >= 128 ? 64 : 32)>(t_base, crow, row < p.M, col0, p, alpha, bias, col_half, EPI_WARPS / 4);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    if (!ok && lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

#include "gemm_pair_kernel.cuh"

template <Kind kKind, int kElemBytes, bool kAMn, bool kBMn, typename TOut>
int launch_variant(const CUtensorMap& tmA, const BMaps& bm, const CUtensorMap& tmC, const GemmParams& p,
                   const Idescs& idescs, Tiling tiling, cudaStream_t stream) {
  const int sms = sm_count();
  const CUtensorMap &tmB = bm.wide, &tmB_pair = bm.half;
  if constexpr (kElemBytes == 2) {
    if (tiling == kSlim) {
      GemmParams q = p;
      q.n_tiles = static_cast<int>((p.N + 63) / 64);
      q.total_tiles = static_cast<int64_t>(q.m_tiles) * q.n_tiles * (p.total_tiles / (static_cast<int64_t>(p.m_tiles) * p.n_tiles));
      auto kern = gemm_tcgen05_kernel<kKind, kElemBytes, kAMn, kBMn, TOut, 64>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      const int grid = static_cast<int>(q.total_tiles < sms ? q.total_tiles : sms);
      launch_overlapped(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tmA, bm.quarter, tmC, q, idescs.slim);
      return check_launch("gemm_tcgen05_kernel (128x64)");
    }
  }
  if (tiling == kSlim) tiling = kNarrow;   // the 64-wide tile exists for 16-bit inputs only
  if (tiling == kPair) {
    auto kern = gemm_tcgen05_pair_kernel<kKind, kElemBytes, kAMn, kBMn, TOut>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PSMEM_BYTES);
    if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int64_t batch = p.total_tiles / (static_cast<int64_t>(p.m_tiles) * p.n_tiles);
    const int64_t pair_tiles = static_cast<int64_t>((p.m_tiles + 1) / 2) * p.n_tiles * batch;
    const int64_t clusters = pair_tiles < sms / 2 ? pair_tiles : sms / 2;
    launch_overlapped(kern, dim3(static_cast<unsigned>(clusters * 2)), dim3(NUM_THREADS), PSMEM_BYTES, stream, tmA, tmB_pair, tmC, p, idescs.pair);
    return check_launch("gemm_tcgen05_pair_kernel");
  }
  if (tiling == kNarrow) {
    // 128x128 tiles: the half-width B box is the one the pair kernel's map already describes
    GemmParams q = p;
    q.n_tiles = static_cast<int>((p.N + 127) / 128);
    q.total_tiles = static_cast<int64_t>(q.m_tiles) * q.n_tiles * (p.total_tiles / (static_cast<int64_t>(p.m_tiles) * p.n_tiles));
    auto kern = gemm_tcgen05_kernel<kKind, kElemBytes, kAMn, kBMn, TOut, 128>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int grid = static_cast<int>(q.total_tiles < sms ? q.total_tiles : sms);
    launch_overlapped(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tmA, tmB_pair, tmC, q, idescs.narrow);
    return check_launch("gemm_tcgen05_kernel (128x128)");
  }
  auto kern = gemm_tcgen05_kernel<kKind, kElemBytes, kAMn, kBMn, TOut, 256>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int grid = static_cast<int>(p.total_tiles < sms ? p.total_tiles : sms);
  launch_overlapped(kern, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, stream, tmA, tmB, tmC, p, idescs.wide);
  return check_launch("gemm_tcgen05_kernel");
}

template <Kind kKind, int kElemBytes, typename TOut>
int launch_layout(int trans_a, int trans_b, const CUtensorMap& tmA, const BMaps& bm, const CUtensorMap& tmC,
                  const GemmParams& p, const Idescs& idescs, Tiling tiling, cudaStream_t s) {
  // trans_a != 0: A is [K, M] row-major -> MN-major operand; trans_b == 0: B is [K, N] -> MN-major.
  if (!trans_a && trans_b)
    return launch_variant<kKind, kElemBytes, false, false, TOut>(tmA, bm, tmC, p, idescs, tiling, s);
  if (!trans_a && !trans_b)
    return launch_variant<kKind, kElemBytes, false, true, TOut>(tmA, bm, tmC, p, idescs, tiling, s);
  if (trans_a && trans_b)
    return launch_variant<kKind, kElemBytes, true, false, TOut>(tmA, bm, tmC, p, idescs, tiling, s);
  return launch_variant<kKind, kElemBytes, true, true, TOut>(tmA, bm, tmC, p, idescs, tiling, s);
}

}  // namespace
}  // namespace kcg
