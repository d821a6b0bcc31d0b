// CTA-pair variant of the tensor-core GEMM (included by gemm_tcgen05.cu inside its
// anonymous namespace).
//
// Two CTAs of a cluster compute one 256x256 tile of C with tcgen05.mma.cta_group::2:
// CTA r of the pair holds rows [128r, 128r+128) of the A tile and of the accumulator, and
// columns [128r, 128r+128) of the B tile; the tensor cores of both SMs read both halves of B.
// Per MMA each SM therefore reads 4 KB of A and 4 KB of B from its own shared memory for
// 128 clocks of work (the single-CTA kernel reads 12 KB), and a stage is 32 KB instead of
// 48 KB, so the ring is 6 deep.  Every load is an ordinary (non-multicast) TMA copy into the
// issuing CTA's own shared memory; only barrier arrivals cross the pair:
//   - TMA completion bytes of both CTAs are counted on the leader's (rank 0) full barrier;
//   - one thread of the leader issues the MMAs and releases ring stages / publishes finished
//     accumulators in both CTAs with a two-CTA tcgen05.commit;
//   - the epilogue warps of both CTAs (eight each, two per lane quarter) hand accumulators back
//     with an mbarrier arrive on the leader's barrier.
#pragma once

constexpr int PSTAGES = 6;
constexpr int PA_BYTES = 128 * 128;           // 128 rows x 128 bytes of K
constexpr int PB_BYTES = 128 * 128;           // this CTA's half of the B tile
constexpr int PSTAGE_BYTES = PA_BYTES + PB_BYTES;
constexpr int PBM = 256, PBN = 256;           // tile of the pair
constexpr int PEPI_STAGE_BYTES = EPI_STAGE_BYTES;   // per epilogue warp: 32 rows x 128 bytes of output
constexpr int PSMEM_BYTES = PSTAGES * PSTAGE_BYTES + 1024 + 256 + EPI_WARPS * PEPI_STAGE_BYTES;

__device__ __forceinline__ void pair_tile_coords(int64_t tile, int m_pairs, int n_tiles, int group_m, int& b, int& mp, int& nt) {
  const int64_t per_batch = static_cast<int64_t>(m_pairs) * n_tiles;
  b = static_cast<int>(tile / per_batch);
  const int r = static_cast<int>(tile % per_batch);
  const int GROUP = max(1, group_m / 2);  // in units of 256-row pairs
  const int group_span = GROUP * n_tiles;
  const int first = (r / group_span) * GROUP;
  const int gsize = min(m_pairs - first, GROUP);
  const int in_group = r % group_span;
  mp = first + in_group % gsize;
  nt = in_group / gsize;
}

template <Kind kKind, int kElemBytes, bool kAMn, bool kBMn, typename TOut>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const GemmParams p, const uint32_t idesc) {
  constexpr int BK = 128 / kElemBytes;
  constexpr int UMMA_K = 32 / kElemBytes;
  constexpr int MN_BOX = 128 / kElemBytes;
  constexpr int MN_BOX_BYTES = BK * 128;
  constexpr int MN_KSTEP = UMMA_K * 128;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* epi_stage = smem + PSTAGES * PSTAGE_BYTES;   // [EPI_WARPS] x 4 KB, 1024-byte aligned like the ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_WARPS * PEPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [PSTAGES]  used in the leader
  uint64_t* empty_bar = bars + PSTAGES;         // [PSTAGES]  one per CTA
  uint64_t* tfull_bar = bars + 2 * PSTAGES;     // [2]        one per CTA
  uint64_t* tempty_bar = bars + 2 * PSTAGES + 2;  // [2]      used in the leader, 8 arrivals
  uint64_t* drain_bar = bars + 2 * PSTAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int64_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int m_pairs = (p.m_tiles + 1) / 2;
  const int64_t total = static_cast<int64_t>(m_pairs) * p.n_tiles * (p.total_tiles / (static_cast<int64_t>(p.m_tiles) * p.n_tiles));

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.c_tma) prefetch_tmap(&tmC);
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();  // after the tensor-memory allocation (the rule in common.cuh)
  grid_dependency_wait();  // set-up done; global memory only after the previous kernel has finished

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0, s = 0, ph = 0;
      bool ok = true;
      for (int64_t tile = cluster_id; tile < total && ok; tile += n_clusters) {
        int b, mp, nt;
        pair_tile_coords(tile, m_pairs, p.n_tiles, p.group_m, b, mp, nt);
        const int m0 = mp * PBM + static_cast<int>(rank) * 128;
        const int n0 = nt * PBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it, ph ^= (s + 1 == PSTAGES), s = (s + 1 == PSTAGES ? 0 : s + 1)) {
          // the first pass over the ring finds every stage free without asking
          if (it >= PSTAGES && !mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* a_dst = smem + s * PSTAGE_BYTES;
          uint8_t* b_dst = a_dst + PA_BYTES;
          // completion bytes of both CTAs go to the leader's barrier
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * PSTAGE_BYTES);
          const uint32_t bar = map_to_cta(&full_bar[s], 0);
          const int k0 = kb * BK;
          if constexpr (!kAMn) {
            tma_load_3d_pair(a_dst, &tmA, bar, k0, m0, b);
          } else if (p.a_blocked && PA_BYTES / MN_BOX_BYTES > 1) {
            tma_load_4d_pair(a_dst, &tmA, bar, 0, k0, m0 / MN_BOX, b);   // all 128-byte column blocks in one copy
          } else {
#pragma unroll
            for (int j = 0; j < PA_BYTES / MN_BOX_BYTES; ++j)
              tma_load_3d_pair(a_dst + j * MN_BOX_BYTES, &tmA, bar, m0 + j * MN_BOX, k0, b);
          }
          if constexpr (!kBMn) {
            tma_load_3d_pair(b_dst, &tmB, bar, k0, n0, b);
          } else if (p.b_blocked && PB_BYTES / MN_BOX_BYTES > 1) {
            tma_load_4d_pair(b_dst, &tmB, bar, 0, k0, n0 / MN_BOX, b);
          } else {
#pragma unroll
            for (int j = 0; j < PB_BYTES / MN_BOX_BYTES; ++j)
              tma_load_3d_pair(b_dst + j * MN_BOX_BYTES, &tmB, bar, n0 + j * MN_BOX, k0, b);
          }
        }
      }
      if (!ok && !*abort_flag) {
        *abort_flag = 1;
        *p.status = KCG_ERR_TIMEOUT;
        __threadfence_system();
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      uint32_t tile_iter = 0;
      bool ok = true;
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t adesc0 = kAMn ? make_smem_desc(smem_base, MN_BOX_BYTES, 1024) : make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = kBMn ? make_smem_desc(smem_base + PA_BYTES, MN_BOX_BYTES, 1024)
                                   : make_smem_desc(smem_base + PA_BYTES, 16, 1024);
      constexpr uint32_t kStageStep = PSTAGE_BYTES >> 4;
      constexpr uint32_t kAStep = (kAMn ? MN_KSTEP : 32) >> 4, kBStep = (kBMn ? MN_KSTEP : 32) >> 4;
      static_assert(BK / UMMA_K == 4, "mma_kblock issues four k-steps");
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      uint32_t s = 0, ph = 0;
      bool ready = false;   // the stage about to be used was seen full by the test issued with the previous k-block
      for (int64_t tile = cluster_id; tile < total && ok; tile += n_clusters, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t d_tmem = tmem_base + acc * PBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!ready && !mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t s1 = s + 1 == PSTAGES ? 0u : s + 1, ph1 = s + 1 == PSTAGES ? ph ^ 1u : ph;
          ready = mma_kblock<kKind, true>(d_tmem, adesc0 + s * kStageStep, bdesc0 + s * kStageStep, kAStep, kBStep, idesc,
                                          kb != 0 ? 1u : 0u, empty0 + s * 8, 3, full0 + s1 * 8, ph1);
          s = s1; ph = ph1;
        }
        if (ok) mma_commit_pair(&tfull_bar[acc], 3);
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit_pair(drain_bar, 1);
        mbar_wait(drain_bar, 0, &zero, 20000000ull);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;
    float alpha = 1.f;
    if (p.scale_a) alpha *= *p.scale_a;
    if (p.scale_b) alpha *= *p.scale_b;
    const TOut* bias = static_cast<const TOut*>(p.bias);
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int64_t tile = cluster_id; tile < total && ok; tile += n_clusters, ++tile_iter) {
      int b, mp, nt;
      pair_tile_coords(tile, m_pairs, p.n_tiles, p.group_m, b, mp, nt);
      const uint32_t acc = tile_iter & 1u, acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(&tfull_bar[acc], acc_ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = static_cast<int64_t>(mp) * PBM + rank * 128 + quarter * 32 + lane;
      const int64_t col0 = static_cast<int64_t>(nt) * PBN;
      TOut* crow = static_cast<TOut*>(p.C) + b * p.stride_c + row * p.ldc;
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * PBN;
      constexpr int VW = Vec16<TOut>::N;
      if (p.n_extra > 0 || p.mc_c != nullptr) {
        // Staged stores: the warp's 32 rows x 128 bytes go through a swizzled shared-memory
        // tile so that eight lanes write one whole 128-byte row segment per instruction —
        // the granularity a store to another GPU's memory should have — and every
        // destination receives the same registers.
        constexpr int RC = 128 / static_cast<int>(sizeof(TOut));   // columns per round
        uint8_t* stg = epi_stage + (warp - 2) * PEPI_STAGE_BYTES;
        const int64_t tile_row0 = static_cast<int64_t>(mp) * PBM + rank * 128 + quarter * 32;
#pragma unroll 1
        for (int c = col_half; c < PBN / RC; c += EPI_WARPS / 4) {
          const int peer0 = p.n_extra > 0 ? static_cast<int>((blockIdx.x + quarter + c) % static_cast<unsigned>(p.n_extra)) : 0;
          uint32_t r[RC];
          if constexpr (RC == 64) tmem_ld64(t_base + c * RC, r); else tmem_ld32(t_base + c * RC, r);
          tmem_wait_ld();
          const int64_t cbase = col0 + c * RC;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            Vec16<TOut> o;
            const int64_t col = cbase + g * VW;
#pragma unroll
            for (int j = 0; j < VW; ++j)
              o.v[j] = col + VW <= p.N ? gemm_epilogue_value<TOut>(__uint_as_float(r[g * VW + j]), alpha, bias, col + j, p.act)
                                       : TOut(0.f);
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((g ^ (lane & 7)) << 4)) = *reinterpret_cast<const uint4*>(&o);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3), ch = lane & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) << 4));
            const int64_t grow = tile_row0 + rr, col = cbase + ch * VW;
            if (grow < p.M && col + VW <= p.N) {
              const int64_t off = b * p.stride_c + grow * p.ldc + col;
              if (p.mc_c != nullptr) {   // one store that NVSwitch delivers to every rank's buffer, this one's included
                multimem_st16(static_cast<TOut*>(p.mc_c) + off, v);
                continue;
              }
              *reinterpret_cast<uint4*>(static_cast<TOut*>(p.C) + off) = v;
              // peers in an order that differs from CTA to CTA and from round to round, so that
              // the stores of the whole grid do not queue up on one NVLink destination at a time
              for (int e = 0; e < p.n_extra; ++e) {
                const int d = (e + peer0) % p.n_extra;
                *reinterpret_cast<uint4*>(static_cast<TOut*>(p.extra_c[d]) + off) = v;
              }
            }
          }
          __syncwarp();
        }
      } else if (p.c_tma) {
        epilogue_rows_tma<TOut, PBN>(t_base, epi_stage + (warp - 2) * PEPI_STAGE_BYTES, &tmC,
                                     mp * PBM + static_cast<int>(rank) * 128 + quarter * 32, static_cast<int>(col0), b, p,
                                     alpha, bias, col_half, EPI_WARPS / 4, lane,
                                     // after the pair's last tile the operand ring is idle: 16 KB of it per warp
                                     tile + n_clusters >= total ? smem + (warp - 2) * 16384 : nullptr);
      } else {
        epilogue_row<TOut, PBN>(t_base, crow, row < p.M, col0, p, alpha, bias, col_half, EPI_WARPS / 4);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&tempty_bar[acc], 0));
    }
    if (!ok && lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  }

  // Neither CTA may leave (or free tensor memory) while the other can still signal it.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}
