// CTA-pair variant of the attention forward kernel (included by fmha_tcgen05.cu inside its
// anonymous namespace; head dimension 128).
//
// Two CTAs of a cluster work on four 128-query tiles with tcgen05.mma.cta_group::2: tile slot i
// (0 or 1) is one M = 256 MMA whose upper 128 rows are CTA 0's tile 2i and whose lower 128 rows
// are CTA 1's tile 2i + 1.  Each CTA stages only HALF of every K and V tile — CTA r holds keys
// [64r, 64r + 64) of K (the N halves of S = Q K^T) and head-dimension columns [64r, 64r + 64) of V
// (the N halves of O += P V) — and the tensor cores of both SMs read both halves.  Per key block
// an SM therefore reads 128 KB of operands from its shared memory and receives 32 KB from TMA,
// against 192 KB + 64 KB in the one-CTA kernel with two tiles, whose MMAs ran at the shared-memory
// bandwidth limit (about 70 instead of 64 clocks each).  Everything else is the two-tile kernel:
//   warps 0-3 / 4-7  softmax warpgroups of this CTA's tile in slot 0 / 1 (one thread per row)
//   warp 8           TMA loader (both CTAs; completion bytes counted on the leader's barriers)
//   warp 9           MMA issuer (one thread of the leader CTA issues for the pair)
// Tensor memory of each CTA: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P overwrites the
// first half of its S.  Every load is an ordinary TMA copy into the issuing CTA's own shared
// memory; only barrier arrivals cross the pair (remote mbarrier.arrive from the peer's softmax
// warps, two-CTA tcgen05.commit from the leader).
#pragma once

constexpr int V3_THREADS = 384;
constexpr int V3_HALF = 16384;   // half of a K or V tile: 64 keys x 128 d, or 128 keys x 64 d (bytes)

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(V3_THREADS, 1)
fmha_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKh,
                     const __grid_constant__ CUtensorMap tmV, const FmhaParams p, const uint32_t idesc_qk,
                     const uint32_t idesc_pv) {
  constexpr int D = 128;
  constexpr int TILE = 2 * TILE16K;   // one 128-row Q tile: two 64-wide blocks of the head dimension
  constexpr int KBLK = 8192;          // one 64-wide block of this CTA's 64 keys of K

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* q_smem = smem;                   // [2][TILE]: this CTA's tiles of slot 0 and slot 1
  uint8_t* kv_smem = smem + 2 * TILE;       // [5][V3_HALF]: ring entry r = (V at 2r, K at 2r + 1), K_0 at 4
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_smem + 5 * V3_HALF);
  uint64_t* q_full = bars;                  // [1]  leader: Q of both CTAs and K_0
  uint64_t* kv_full = bars + 1;             // [2]  leader
  uint64_t* kv_empty = bars + 3;            // [2]  each CTA (two-CTA commit)
  uint64_t* s_full = bars + 5;              // [2]  each CTA (two-CTA commit)
  uint64_t* p_full = bars + 7;              // [2 slots][2 halves]  leader, 8 arrivals (4 warps x 2 CTAs)
  uint64_t* drain_bar = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int quads = (p.q_tiles + 3) / 4;
  const int cid = static_cast<int>(blockIdx.x >> 1);
  const int qd = p.causal ? (quads - 1 - cid) : cid;   // causal: the longest quads start first
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qd * 4 * BM;
  const int off = p.Skv - p.Sq;
  // key blocks of the two slots: what the later tile of the slot (CTA 1's) needs; CTA 0's tile sees
  // its last block or two fully masked
  const int kv_end0 = p.causal ? min(p.Skv, q0 + 2 * BM + off) : p.Skv;
  const int kv_end1 = p.causal ? min(p.Skv, q0 + 4 * BM + off) : p.Skv;
  const int n_blk0 = kv_end0 > 0 ? (kv_end0 + BN - 1) / BN : 0;
  const int n_blk1 = kv_end1 > 0 ? (kv_end1 + BN - 1) / BN : 0;
  const int n_max = max(n_blk0, n_blk1);

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmKh);
    prefetch_tmap(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[2 * s], 8);
      mbar_init(&p_full[2 * s + 1], 8);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();  // after the tensor-memory allocation (the rule in common.cuh)
  grid_dependency_wait();    // set-up done; global memory only after the previous kernel has finished

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA loader (both CTAs)
    reg_dealloc<V2_REGS_SERVICE>();
    if (lane == 0 && n_max > 0) {
      bool ok = true;
      const int r64 = static_cast<int>(rank) * 64;
      if (rank == 0) mbar_expect_tx(q_full, 2 * (2 * TILE + V3_HALF));
      const uint32_t bar_q = map_to_cta(q_full, 0);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int d = 0; d < 2; ++d)
          tma_load_4d_pair(q_smem + i * TILE + d * TILE16K, &tmQ, bar_q, d * 64, q0 + (2 * i + static_cast<int>(rank)) * BM, h, b);
#pragma unroll
      for (int d = 0; d < 2; ++d) tma_load_4d_pair(kv_smem + 4 * V3_HALF + d * KBLK, &tmKh, bar_q, d * 64, r64, h, b);
      for (int j = 0; j < n_max; ++j) {
        const uint32_t r = j & 1u, ph = (j >> 1) & 1u;
        if (!mbar_wait(&kv_empty[r], ph ^ 1u, abort_flag)) { ok = false; break; }
        const bool more = j + 1 < n_max;
        if (rank == 0) mbar_expect_tx(&kv_full[r], 2 * (more ? 2 * V3_HALF : V3_HALF));
        const uint32_t bar = map_to_cta(&kv_full[r], 0);
        // this CTA's 64 head-dimension columns of V_j: one 128-key x 128-byte block
        tma_load_4d_pair(kv_smem + (2 * r) * V3_HALF, &tmV, bar, r64, j * BN, h, b);
        if (more) {
#pragma unroll
          for (int d = 0; d < 2; ++d)
            tma_load_4d_pair(kv_smem + (2 * r + 1) * V3_HALF + d * KBLK, &tmKh, bar, d * 64, (j + 1) * BN + r64, h, b);
        }
      }
      if (!ok && !*abort_flag) {
        *abort_flag = 1;
        *p.status = KCG_ERR_TIMEOUT;
        __threadfence_system();
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    reg_dealloc<V2_REGS_SERVICE>();
    if (lane == 0 && rank == 0 && n_max > 0) {
      bool ok = true;
      const uint64_t q_desc0 = make_smem_desc(smem_u32(q_smem), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc(smem_u32(kv_smem), 16, 1024);        // K halves (K-major)
      const uint64_t v_desc0 = make_smem_desc(smem_u32(kv_smem), TILE16K, 1024);   // V halves (MN-major, one column block)
      auto issue_s = [&](int i, int j) {  // S_i(j) = Q_i K_j^T for both CTAs' tiles of slot i
        const uint64_t qd_ = q_desc0 + static_cast<uint64_t>((i * TILE) >> 4);
        const uint64_t kd = k_desc0 + static_cast<uint64_t>(((j == 0 ? 4 : 2 * ((j - 1) & 1) + 1) * V3_HALF) >> 4);
#pragma unroll
        for (int d = 0; d < 2; ++d)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss_pair<Kind::F16>(tmem_base + i * BN, qd_ + ((d * TILE16K + k * 32) >> 4), kd + ((d * KBLK + k * 32) >> 4),
                                   idesc_qk, (d | k) != 0 ? 1u : 0u);
      };
      auto issue_pv = [&](int i, int j, int half) {  // O_i += P_i(j)[:, half] V_j[half, :]
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((2 * (j & 1) * V3_HALF) >> 4);
#pragma unroll
        for (int kk = half * 4; kk < half * 4 + 4; ++kk)
          mma_ts_f16_pair(tmem_base + 256 + i * BN, tmem_base + i * BN + kk * 8, vd + ((kk * 2048) >> 4), idesc_pv,
                          (j | kk) != 0 ? 1u : 0u);
      };
      ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if ((i == 0 ? n_blk0 : n_blk1) > 0) {
            issue_s(i, 0);
            mma_commit_pair(&s_full[i], 3);
          }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        ok = mbar_wait(&kv_full[j & 1], (j >> 1) & 1u, abort_flag);
        if (!ok) break;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int n_i = i == 0 ? n_blk0 : n_blk1;
          if (j >= n_i) continue;
          ok = mbar_wait_cluster(&p_full[2 * i], j & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_pv(i, j, 0);
          ok = mbar_wait_cluster(&p_full[2 * i + 1], j & 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_pv(i, j, 1);
          if (j + 1 < n_i) issue_s(i, j + 1);
          mma_commit_pair(&s_full[i], 3);   // the next score tile, or the finished output, in both CTAs
        }
        if (ok) mma_commit_pair(&kv_empty[j & 1], 3);
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit_pair(drain_bar, 1);
        mbar_wait(drain_bar, 0, &zero, 20000000ull);
      }
    }
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax / epilogue (both CTAs)
    reg_alloc<V2_REGS_SOFTMAX>();
    const int i = warp >> 2;                      // tile slot of this warpgroup
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int tile_row0 = q0 + (2 * i + static_cast<int>(rank)) * BM;
    const int qi = tile_row0 + r;
    const float c = p.scale_log2;
    const int n_mine = i == 0 ? n_blk0 : n_blk1;
    const uint32_t s_addr = tmem_base + lane_base + i * BN;
    const uint32_t o_addr = tmem_base + lane_base + 256 + i * BN;
    const uint32_t p_bar0 = map_to_cta(&p_full[2 * i], 0), p_bar1 = map_to_cta(&p_full[2 * i + 1], 0);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait(&s_full[i], j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BN;
      int limit = p.Skv - kv0;
      if (p.causal) limit = min(limit, qi + off + 1 - kv0);
      softmax_block<T, D>(s_addr, o_addr, j, limit, c, m, l, lane,
                          [&](int half) { mbar_arrive_cluster_relaxed(half ? p_bar1 : p_bar0); });
    }
    // epilogue: the commit after the last PV arrives on s_full once more
    if (ok && n_mine > 0) ok = mbar_wait(&s_full[i], n_mine & 1u, abort_flag);
    if (ok) {
      tc_fence_after();
      store_output<T, D>(p, o_addr, n_mine > 0, l, b, h, tile_row0 + quarter * 32, lane,
                         q_smem + i * TILE + quarter * (32 * D * 2), static_cast<int>(blockIdx.x + blockIdx.y) + warp);
    } else if (lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  } else {
    reg_dealloc<V2_REGS_SERVICE>();   // warps 10-11: only the register hand-over
  }

  // Neither CTA may leave (or free tensor memory) while the other can still signal it.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <typename T>
int launch_fmha_pair(const CUtensorMap& tmQ, const CUtensorMap& tmKh, const CUtensorMap& tmV, const FmhaParams& p,
                     uint32_t fmt, cudaStream_t stream) {
  constexpr int SMEM = 2 * (2 * TILE16K) + 5 * V3_HALF + 1024 + 256;
  auto kern = fmha_fwd_pair_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "fmha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, 2 * BM, BN);
  const uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, 2 * BM, 128);
  dim3 grid(2 * ((p.q_tiles + 3) / 4), p.B * p.H);
  launch_overlapped(kern, grid, dim3(V3_THREADS), SMEM, stream, tmQ, tmKh, tmV, p, idesc_qk, idesc_pv);
  return check_launch("fmha_fwd_pair_kernel");
}
