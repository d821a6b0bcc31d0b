// CTA-pair attention kernel with two score buffers per tile, whose two softmax warpgroups take
// alternate key blocks (included by fmha_tcgen05.cu inside its anonymous namespace; head dimension 128).
//
// In the two-tile kernels the per-tile chain  softmax -> P -> PV -> next S -> softmax  sets the
// pace: the score buffer of a tile cannot be refilled before its P (which overwrites it) has been
// consumed.  Here a CTA owns ONE 128-query tile, which leaves tensor memory for two score buffers
// (S_a, S_b, 128 columns each) and two P buffers (64 columns each) next to the output accumulator;
// a score buffer is refilled as soon as its row values have been read into registers, so S(j+1)
// and S(j+2) are computed while block j is in its softmax.  Warpgroup 0 takes the even key blocks (buffer a), warpgroup 1 the
// odd ones (buffer b); thread t of either warpgroup owns query row t, so a row is served by two
// threads that work one block apart, each with two block times for its softmax, and their
// special-function phases interleave instead of coinciding.  What the online softmax carries from
// block to block is shared: the row's reference maximum travels through shared memory (mref, one
// small barrier per block: a thread decides about block j only after the decision about block
// j - 1 has been published, which happens early in that block's softmax), each thread keeps the
// partial row sum of its own blocks relative to the reference and rescales it when the reference
// has moved, and whoever moves the reference rescales the accumulator once no MMA is in flight on
// it.  Two such CTAs form a pair (tcgen05 cta_group::2): CTA r holds query tile 2c + r, keys
// [64r, 64r + 64) of every K tile and head-dimension columns [64r, 64r + 64) of every V tile, which
// halves the operand bytes an SM stages and reads.
//   warps 0-3   softmax warpgroup 0: key blocks 0, 2, 4, ...
//   warps 4-7   softmax warpgroup 1: key blocks 1, 3, 5, ...
//   warp 8      TMA loader (both CTAs): Q, K_0, K_1, then (V_j, K_{j+2}) per key block, ring of 3
//   warp 9      MMA issuer (leader CTA) of the scores:  S(j+2) = Q K_{j+2}^T as soon as S(j) has been read
//   warp 10     MMA issuer (leader CTA) of the output:  O += P(j) V_j
// Every load is an ordinary TMA copy into the issuing CTA's own shared memory.
#pragma once

constexpr int V5_THREADS = 384;
constexpr int V5_RING = 3;

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(V5_THREADS, 1)
fmha_fwd_split_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKh,
                      const __grid_constant__ CUtensorMap tmV, const FmhaParams p, const uint32_t idesc_qk,
                      const uint32_t idesc_pv) {
  constexpr int D = 128;
  constexpr int TILE = 2 * TILE16K;   // the 128-row Q tile
  constexpr int HALF = V3_HALF;       // half of a K or V tile (16 KB)
  constexpr int KBLK = 8192;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* q_smem = smem;                        // [TILE]
  uint8_t* k01_smem = smem + TILE;               // [2][HALF]  K_0 and K_1 (never reused)
  uint8_t* ring_smem = k01_smem + 2 * HALF;      // [V5_RING][2][HALF]  entry = (V_j, K_{j+2})
  float* mref = reinterpret_cast<float*>(ring_smem + V5_RING * 2 * HALF);   // [128 rows]  the rows' reference maxima
  float* xsum = mref + 128;                      // [2 warpgroups][128 rows]  final partial row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(xsum + 2 * 128);
  uint64_t* q_full = bars;                       // [1]  leader: Q of both CTAs, K_0, K_1
  uint64_t* kv_full = bars + 1;                  // [3]  leader
  uint64_t* s_full = bars + 7;                   // [2 buffers]  each CTA (two-CTA commit)
  uint64_t* p_full = bars + 9;                   // [2 buffers]  leader, 8 arrivals (4 warps x 2 CTAs): all of P(j)
  uint64_t* s_free = bars + 11;                  // [2 buffers]  leader, 8 arrivals: S(j) has been read by all its threads
  uint64_t* pv_done = bars + 4;                  // [2 buffers]  each CTA (two-CTA commit) after PV(j), j & 1 = buffer
  uint64_t* o_done = bars + 13;                  // [1]  each CTA (two-CTA commit) after the last PV
  uint64_t* drain_bar = bars + 23;               // [2]  one per issuing thread
  uint64_t* row_sync = bars + 15;                // [4 quarters]  each CTA, 1 arrival: block j's reference is published
  uint64_t* fin_sync = bars + 19;                // [4 quarters]  each CTA, 2 arrivals: both partial row sums are there
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pairs = (p.q_tiles + 1) / 2;
  const int cid = static_cast<int>(blockIdx.x >> 1);
  const int pr = p.causal ? (pairs - 1 - cid) : cid;   // causal: the longest pairs start first
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = pr * 2 * BM;
  const int off = p.Skv - p.Sq;
  // key blocks: what the later tile of the pair (CTA 1's) needs; CTA 0 may see its last block fully masked
  const int kv_end = p.causal ? min(p.Skv, q0 + 2 * BM + off) : p.Skv;
  const int n_blk = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmKh);
    prefetch_tmap(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < V5_RING; ++s) {
      mbar_init(&kv_full[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);
      mbar_init(&s_free[s], 8);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(o_done, 1);
    mbar_init(&drain_bar[0], 1);
    mbar_init(&drain_bar[1], 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&row_sync[s], 1);
      mbar_init(&fin_sync[s], 2);
    }
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
    if (lane == 0 && n_blk > 0) {
      bool ok = true;
      const int r64 = static_cast<int>(rank) * 64;
      const int n_k01 = n_blk > 1 ? 2 : 1;
      if (rank == 0) mbar_expect_tx(q_full, 2 * (TILE + n_k01 * HALF));
      const uint32_t bar_q = map_to_cta(q_full, 0);
#pragma unroll
      for (int d = 0; d < 2; ++d) tma_load_4d_pair(q_smem + d * TILE16K, &tmQ, bar_q, d * 64, q0 + static_cast<int>(rank) * BM, h, b);
      for (int t = 0; t < n_k01; ++t)
#pragma unroll
        for (int d = 0; d < 2; ++d) tma_load_4d_pair(k01_smem + t * HALF + d * KBLK, &tmKh, bar_q, d * 64, t * BN + r64, h, b);
      for (int j = 0; j < n_blk; ++j) {
        const uint32_t e = j % V5_RING;
        // Entry e last held (V_{j-3}, K_{j-1}); its readers are PV(j-3) and S(j-1), issued by two
        // threads, each followed by a commit: pv_done and s_full.  (A barrier's phases have to be
        // waited for in order: the loader passes every phase of pv_done, and of s_full once it has
        // passed S(0) and S(1).)
        if (j == V5_RING && !(mbar_wait(&s_full[0], 0, abort_flag) && mbar_wait(&s_full[1], 0, abort_flag))) { ok = false; break; }
        if (j >= V5_RING && !(mbar_wait(&pv_done[(j - 3) & 1], ((j - 3) >> 1) & 1u, abort_flag) &&
                              mbar_wait(&s_full[(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_flag))) { ok = false; break; }
        const bool more = j + 2 < n_blk;
        if (rank == 0) mbar_expect_tx(&kv_full[e], 2 * (more ? 2 * HALF : HALF));
        const uint32_t bar = map_to_cta(&kv_full[e], 0);
        uint8_t* ent = ring_smem + e * 2 * HALF;
        tma_load_4d_pair(ent, &tmV, bar, r64, j * BN, h, b);   // this CTA's 64 columns of V_j
        if (more) {
#pragma unroll
          for (int d = 0; d < 2; ++d) tma_load_4d_pair(ent + HALF + d * KBLK, &tmKh, bar, d * 64, (j + 2) * BN + r64, h, b);
        }
      }
      if (!ok && !*abort_flag) {
        *abort_flag = 1;
        *p.status = KCG_ERR_TIMEOUT;
        __threadfence_system();
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers (leader only)
    // Two threads issue: warp 9 the score MMAs S(j) = Q K_j^T, warp 10 the output MMAs O += P(j) V_j.
    // The two streams are independent (different accumulators, different operands), and around
    // its eight MMAs per block each thread spends a few hundred clocks on barrier waits, the
    // tcgen05 fence and the commit; with a single thread the tensor pipe sat idle during those
    // (measured: 1950 clocks per key block for 1024 clocks of MMA, every wait already satisfied).
    reg_dealloc<V2_REGS_SERVICE>();
    if (lane == 0 && rank == 0 && n_blk > 0) {
      bool ok = true;
      if (warp == 9) {
        const uint64_t q_desc0 = make_smem_desc(smem_u32(q_smem), 16, 1024);
        const uint64_t k01_desc0 = make_smem_desc(smem_u32(k01_smem), 16, 1024);
        const uint64_t kr_desc0 = make_smem_desc(smem_u32(ring_smem) + HALF, 16, 1024);    // K half of ring entry 0
        auto issue_s = [&](int j) {  // S(j) = Q K_j^T into buffer j & 1
          const uint64_t kd = j < 2 ? k01_desc0 + static_cast<uint64_t>((j * HALF) >> 4)
                                    : kr_desc0 + static_cast<uint64_t>((((j - 2) % V5_RING) * 2 * HALF) >> 4);
#pragma unroll
          for (int d = 0; d < 2; ++d)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss_pair<Kind::F16>(tmem_base + (j & 1) * BN, q_desc0 + ((d * TILE16K + k * 32) >> 4),
                                     kd + ((d * KBLK + k * 32) >> 4), idesc_qk, (d | k) != 0 ? 1u : 0u);
        };
        ok = mbar_wait(q_full, 0, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_s(0);
          mma_commit_pair(&s_full[0], 3);
          if (n_blk > 1) {
            issue_s(1);
            mma_commit_pair(&s_full[1], 3);
          }
        }
        // S(j+2) as soon as K_{j+2} has landed and the softmax threads have read S(j) out of its
        // buffer, which they do long before they deliver P(j)
        for (int j = 0; j + 2 < n_blk && ok; ++j) {
          const int bsel = j & 1;
          if (!mbar_wait(&kv_full[j % V5_RING], (j / V5_RING) & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait_cluster(&s_free[bsel], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 2);
          mma_commit_pair(&s_full[bsel], 3);
        }
      } else {
        const uint64_t v_desc0 = make_smem_desc(smem_u32(ring_smem), TILE16K, 1024);       // V half of ring entry 0
        for (int j = 0; j < n_blk && ok; ++j) {
          const int bsel = j & 1;
          if (!mbar_wait(&kv_full[j % V5_RING], (j / V5_RING) & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait_cluster(&p_full[bsel], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t vd = v_desc0 + static_cast<uint64_t>(((j % V5_RING) * 2 * HALF) >> 4);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)   // O += P(j) V_j
            mma_ts_f16_pair(tmem_base + 256, tmem_base + 384 + bsel * 64 + kk * 8, vd + ((kk * 2048) >> 4), idesc_pv,
                            (j | kk) != 0 ? 1u : 0u);
          mma_commit_pair(&pv_done[bsel], 3);
        }
        if (ok) mma_commit_pair(o_done, 3);
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit_pair(&drain_bar[warp - 9], 1);
        mbar_wait(&drain_bar[warp - 9], 0, &zero, 20000000ull);
      }
    }
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax / epilogue (both CTAs)
    reg_alloc<V2_REGS_SOFTMAX>();
    const int g = warp >> 2;                      // this warpgroup takes key blocks j = g, g + 2, ...
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + static_cast<int>(rank) * BM + r;
    const float c = p.scale_log2;
    const uint32_t s_addr = tmem_base + lane_base + g * BN;   // buffer g holds this warpgroup's blocks
    const uint32_t o_all = tmem_base + lane_base + 256;       // the row's 128 output columns
    const uint32_t p_addr = tmem_base + lane_base + 384 + g * 64;   // this warpgroup's P buffer
    const uint32_t p_bar = map_to_cta(&p_full[g], 0), s_free_bar = map_to_cta(&s_free[g], 0);
    // m is the reference maximum the row's exponentials are taken against.  It is shared by the two
    // threads of a row through mref[]: the thread handling block j takes over the value left by
    // block j - 1 (row_sync orders the two), decides whether block j moves it, publishes it, and
    // only then goes on to its exponentials, which overlap the other thread's next block.
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = g; j < n_blk; j += 2) {
      if (!mbar_wait(&s_full[g], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (j > 0) {
        if (!mbar_wait(&row_sync[quarter], (j - 1) & 1u, abort_flag)) { ok = false; break; }
        const float m_now = mref[r];
        if (m_now != m) {   // the other thread moved the reference: this thread's partial row sum follows
          l = (m == -INFINITY) ? 0.f : l * fast_exp2(m - m_now);
          m = m_now;
        }
      }
      const int kv0 = j * BN;
      int limit = p.Skv - kv0;
      if (p.causal) limit = min(limit, qi + off + 1 - kv0);
      ok = softmax_block_px<T, D>(
          s_addr, o_all, p_addr, j, limit, c, m, l, lane,
          [&]() { mbar_arrive_cluster_relaxed(s_free_bar); },   // S(j) is in registers: its buffer may be refilled
          [&]() {   // this block's reference is final: hand it to the thread that takes block j + 1
            mref[r] = m;
            __syncwarp();
            if (lane == 0) mbar_arrive(&row_sync[quarter]);
          },
          [&]() { return mbar_wait(&pv_done[1 - g], ((j - 1) >> 1) & 1u, abort_flag); },   // O holds block j - 1
          [&]() { return j < 2 || mbar_wait(&pv_done[g], ((j - 2) >> 1) & 1u, abort_flag); },   // P(j-2) has been consumed
          [&]() { mbar_arrive_cluster_relaxed(p_bar); });
      if (!ok) break;
    }
    // epilogue: all of O is there once the last PV has finished.  The two threads of a row bring
    // their partial sums to the final reference and add them; each stores 64 of the 128 columns.
    if (ok && n_blk > 0) ok = mbar_wait(o_done, 0, abort_flag);
    if (ok && n_blk > 0) {
      // the last decision was published by the thread that took block n_blk - 1
      if (((n_blk - 1) & 1) != g) ok = mbar_wait(&row_sync[quarter], (n_blk - 1) & 1u, abort_flag);
    }
    if (ok) {
      tc_fence_after();
      float lt = 0.f;
      if (n_blk > 0) {
        const float m_fin = mref[r];
        const float mine = (m == -INFINITY || l == 0.f) ? 0.f : l * fast_exp2(m - m_fin);
        xsum[g * 128 + r] = mine;
        __syncwarp();
        if (lane == 0) mbar_arrive(&fin_sync[quarter]);
        ok = mbar_wait(&fin_sync[quarter], 0, abort_flag);
        lt = mine + xsum[(1 - g) * 128 + r];
      }
      const float inv_l = lt > 0.f ? 1.0f / lt : 0.f;
      const uint32_t o_addr = o_all + g * 64;
      T* orow = static_cast<T*>(p.O) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh +
                static_cast<int64_t>(qi) * p.o_ss + g * 64;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t oreg[32];
        if (n_blk > 0) {
          tmem_ld32(o_addr + cc * 32, oreg);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) oreg[k] = 0u;
        }
        if (qi < p.Sq && ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack2<T>(__uint_as_float(oreg[q * 8 + 0]) * inv_l, __uint_as_float(oreg[q * 8 + 1]) * inv_l);
            o.y = pack2<T>(__uint_as_float(oreg[q * 8 + 2]) * inv_l, __uint_as_float(oreg[q * 8 + 3]) * inv_l);
            o.z = pack2<T>(__uint_as_float(oreg[q * 8 + 4]) * inv_l, __uint_as_float(oreg[q * 8 + 5]) * inv_l);
            o.w = pack2<T>(__uint_as_float(oreg[q * 8 + 6]) * inv_l, __uint_as_float(oreg[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + cc * 32 + q * 8) = o;
          }
        }
      }
    }
    if (!ok && lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  } else {
    reg_dealloc<V2_REGS_SERVICE>();   // warp 11: only the register hand-over
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
int launch_fmha_split(const CUtensorMap& tmQ, const CUtensorMap& tmKh, const CUtensorMap& tmV, const FmhaParams& p,
                      uint32_t fmt, cudaStream_t stream) {
  constexpr int SMEM = 2 * TILE16K + 2 * V3_HALF + V5_RING * 2 * V3_HALF + (128 + 2 * 128) * 4 + 1024 + 256;
  auto kern = fmha_fwd_split_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "fmha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, 2 * BM, BN);
  const uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, 2 * BM, 128);
  dim3 grid(2 * ((p.q_tiles + 1) / 2), p.B * p.H);
  launch_overlapped(kern, grid, dim3(V5_THREADS), SMEM, stream, tmQ, tmKh, tmV, p, idesc_qk, idesc_pv);
  return check_launch("fmha_fwd_split_kernel");
}
