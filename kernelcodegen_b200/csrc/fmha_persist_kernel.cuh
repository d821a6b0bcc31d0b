// Persistent form of the two-tile attention kernel (included by fmha_tcgen05.cu inside its
// anonymous namespace; variant 5 of kcg_fmha_set_p_in_tmem).
//
// The two-tile kernel launches one CTA per (pair of query tiles, batch x head).  Only one such
// CTA fits an SM (224 KB of shared memory, all 512 tensor-memory columns), so nothing hides a
// CTA's start-up — barrier set-up, tensor-memory allocation, the Q / K_0 load, the first
// QK^T and the first softmax — nor its output store: about 5 us per CTA during which the tensor
// pipe idles, a quarter of the run time at S = 1024.  Here a CTA stays resident and walks over
// work items (grid = a number of CTAs close to the SM count, items dealt round-robin):
//   - the loader fetches Q and K_0 of the next item as soon as the last QK^T of the current
//     item has completed (q_empty), i.e. under the current item's last softmax and PV;
//   - the MMA thread issues the next item's first QK^T right behind the current item's last
//     PV, so those scores are ready when the softmax warps return from storing the output;
//   - the softmax warps release the output accumulator (o_free) as soon as they have read it and
//     send the rows out through TMA stores, staged in the K / V ring entry that is idle at the
//     end of an item; the loader refills that entry only when all eight warps are done (stage_done);
//   - every barrier keeps running across items: phases are counted, not derived from the
//     key-block index.
// Items are numbered head-major (the pairs of one head are adjacent, so CTAs working on the same
// head at the same time share its K / V through L2); for a causal mask the pairs of a head run
// longest first, and grid size and dealing order are chosen so that every CTA gets a fair mix
// of pair lengths (persist_plan).
#pragma once

// The issuing thread carries more state across items than in the one-item kernel (phase counters of
// every barrier, the item's coordinates): 104 registers for the service warps, 200 for the softmax warps.
// setmaxnreg only redistributes the registers the CTA was launched with (384 threads x 168): a split
// that adds up to more makes the raising warps wait for registers that never come.
constexpr int V2P_REGS_SOFTMAX = 200, V2P_REGS_SERVICE = 104;
static_assert(2 * 128 * V2P_REGS_SOFTMAX + 128 * V2P_REGS_SERVICE <= V2_THREADS * 168, "register split exceeds the CTA's allocation");

template <typename T, int D>
__global__ void __launch_bounds__(V2_THREADS, 1)
fmha_fwd_kernel2p(const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FmhaParams p, const uint32_t idesc_qk,
                  const uint32_t idesc_pv, const int snake) {
  constexpr int DB = D / 64;
  constexpr int TILE = DB * TILE16K;   // bytes of one Q, K or V tile
  constexpr int NSLOT = 5;             // two (V, K) ring entries plus the slot of K_0

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* q_smem = smem;                   // [2][TILE]
  uint8_t* kv_smem = smem + 2 * TILE;       // [NSLOT][TILE]
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_smem + NSLOT * TILE);
  uint64_t* q_full = bars;                  // [1]
  uint64_t* q_empty = bars + 1;             // [1]  the item's last QK^T has read Q (and K_0 long before)
  uint64_t* kv_full = bars + 2;             // [2]
  uint64_t* kv_empty = kv_full + 2;         // [2]
  uint64_t* s_full = kv_empty + 2;          // [2]
  uint64_t* p_full = s_full + 2;            // [2 tiles][2 column halves]
  uint64_t* o_free = p_full + 4;            // [2]  the tile's output accumulator has been read out
  // [2]  the item's last PV of the tile has completed.  (In the one-item kernel this signal shares
  // s_full; here the next item's first score tile may complete right behind it, and a waiter
  // that has not yet looked at a barrier must never fall two phases behind it.)
  uint64_t* o_full = o_free + 2;
  // [1]  all eight softmax warps have stored the item's output: the ring entry they staged it in
  // (the one the item's second-to-last key block used) may receive the next item's first K / V
  uint64_t* stage_done = o_full + 2;
  uint64_t* drain_bar = stage_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = (p.q_tiles + 1) / 2;
  const int items = pairs * p.B * p.H;
  const int off = p.Skv - p.Sq;

  // Work item k -> batch, head, first query row, key blocks of the two tiles.
  struct Item { int b, h, q0, n0, n1, nmax; };
  auto decode = [&](int k) {
    Item it;
    const int bh = k / pairs, pos = k % pairs;
    const int pr = p.causal ? pairs - 1 - pos : pos;
    it.b = bh / p.H; it.h = bh % p.H;
    it.q0 = pr * 2 * BM;
    const int kv_end0 = p.causal ? min(p.Skv, it.q0 + BM + off) : p.Skv;
    const int kv_end1 = p.causal ? min(p.Skv, it.q0 + 2 * BM + off) : p.Skv;
    it.n0 = kv_end0 > 0 ? (kv_end0 + BN - 1) / BN : 0;
    it.n1 = kv_end1 > 0 ? (kv_end1 + BN - 1) / BN : 0;
    it.nmax = max(it.n0, it.n1);
    return it;
  };

  // This CTA's item of round r (items are dealt in rounds of gridDim.x): in the plain order CTA c
  // takes item r * G + c; in the snake order every second round runs backwards, so that with a
  // grid that is a multiple of the pairs per head a CTA alternates between a pair position and its
  // mirror image (the longest and the shortest pair of a causal head, and so on).
  auto item_of_round = [&](int r) {
    const int c = (snake && (r & 1)) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
    return r * static_cast<int>(gridDim.x) + c;
  };

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 4);
      mbar_init(&p_full[2 * i + 1], 4);
      mbar_init(&o_free[i], 4);
      mbar_init(&o_full[i], 1);
    }
    mbar_init(stage_done, 8);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();  // after the tensor-memory allocation (the rule in common.cuh)
  grid_dependency_wait();  // set-up done; global memory only after the previous kernel has finished

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA loader
    reg_dealloc<V2P_REGS_SERVICE>();
    if (lane == 0) {
      bool ok = true;
      uint32_t n_item = 0;   // items with key blocks loaded so far
      uint32_t g = 0;        // ring entries filled so far
      for (int rd = 0; rd * static_cast<int>(gridDim.x) < items && ok; ++rd) {
        const int k = item_of_round(rd);
        if (k >= items) continue;
        const Item it = decode(k);
        if (it.nmax == 0) continue;
        // Q of both tiles and K_0: free once the previous item's last QK^T has completed
        if (n_item > 0 && !mbar_wait(q_empty, (n_item - 1) & 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(q_full, 3 * TILE);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int d = 0; d < DB; ++d)
            tma_load_4d(q_smem + i * TILE + d * TILE16K, &tmQ, q_full, d * 64, it.q0 + i * BM, it.h, it.b);
#pragma unroll
        for (int d = 0; d < DB; ++d) tma_load_4d(kv_smem + 4 * TILE + d * TILE16K, &tmK, q_full, d * 64, 0, it.h, it.b);
        ++n_item;
        // one ring entry per key block j: V_j (slot 2r) and K_{j+1} (slot 2r+1), r = entry & 1
        for (int j = 0; j < it.nmax; ++j, ++g) {
          const uint32_t r = g & 1u, ph = (g >> 1) & 1u;
          if (g >= 2 && !mbar_wait(&kv_empty[r], ph ^ 1u, abort_flag)) { ok = false; break; }
          // the previous item's output was staged in this ring entry on its way to global memory
          if (j == 0 && n_item > 1 && !mbar_wait(stage_done, (n_item - 2) & 1u, abort_flag)) { ok = false; break; }
          const bool more = j + 1 < it.nmax;
          mbar_expect_tx(&kv_full[r], more ? 2 * TILE : TILE);
#pragma unroll
          for (int d = 0; d < DB; ++d)
            tma_load_4d(kv_smem + (2 * r) * TILE + d * TILE16K, &tmV, &kv_full[r], d * 64, j * BN, it.h, it.b);
          if (more) {
#pragma unroll
            for (int d = 0; d < DB; ++d)
              tma_load_4d(kv_smem + (2 * r + 1) * TILE + d * TILE16K, &tmK, &kv_full[r], d * 64, (j + 1) * BN, it.h, it.b);
          }
        }
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        // let the copies that were issued land before the CTA goes away
        int zero = 0;
        if (n_item > 0) mbar_wait(q_full, (n_item - 1) & 1u, &zero, 2000000ull);
        for (uint32_t u = g > 2 ? g - 2 : 0; u < g; ++u) mbar_wait(&kv_full[u & 1], (u >> 1) & 1u, &zero, 2000000ull);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    reg_dealloc<V2P_REGS_SERVICE>();
    if (lane == 0) {
      bool ok = true;
      const uint32_t q_addr = smem_u32(q_smem);
      const uint64_t q_desc0 = make_smem_desc(q_addr, 16, 1024);
      const uint64_t kv_desc0 = make_smem_desc(smem_u32(kv_smem), 16, 1024);          // K tiles (K-major)
      const uint64_t v_desc0 = make_smem_desc(smem_u32(kv_smem), TILE16K, 1024);      // V tiles (MN-major)
      const uint64_t k0_desc = kv_desc0 + static_cast<uint64_t>((4 * TILE) >> 4);
      auto issue_s0 = [&](int i) {  // S_i(0) = Q_i K_0^T
        const uint64_t qd = q_desc0 + static_cast<uint64_t>((i * TILE) >> 4);
#pragma unroll
        for (int d = 0; d < DB; ++d)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss<Kind::F16>(tmem_base + i * BN, qd + ((d * TILE16K + k * 32) >> 4), k0_desc + ((d * TILE16K + k * 32) >> 4),
                              idesc_qk, (d | k) != 0 ? 1u : 0u);
      };
      const uint32_t kvf0 = smem_u32(kv_full), pf0 = smem_u32(p_full), sf0 = smem_u32(s_full), of0 = smem_u32(o_full);
      uint32_t n_item = 0;            // items started
      uint32_t g = 0;                 // ring entries consumed
      uint32_t cp0 = 0, cp1 = 0;      // P blocks consumed per tile (phase counters of p_full)
      uint32_t co0 = 0, co1 = 0;      // items whose output accumulator this tile has produced (o_free phases)
      // Barriers already seen complete by a test that rode along with an earlier MMA batch
      bool r_kv = false, r_p00 = false, r_p01 = false, r_p10 = false, r_p11 = false;
      for (int rd = 0; rd * static_cast<int>(gridDim.x) < items && ok; ++rd) {
        const int k = item_of_round(rd);
        if (k >= items) continue;
        const Item it = decode(k);
        if (it.nmax == 0) continue;
        if (!mbar_wait(q_full, n_item & 1u, abort_flag)) { ok = false; break; }
        ++n_item;
        tc_fence_after();
        // first score tiles: the tensor-memory columns are free (the previous item's last P of
        // this tile has been consumed by a PV issued earlier by this thread)
        if (it.n0 > 0) { issue_s0(0); mma_commit(&s_full[0]); }
        if (it.n1 > 0) { issue_s0(1); mma_commit(&s_full[1]); }
        if (it.nmax == 1) mma_commit(q_empty);
        for (int j = 0; j < it.nmax && ok; ++j, ++g) {
          const uint32_t r = g & 1u;
          if (!r_kv && !mbar_wait(&kv_full[r], (g >> 1) & 1u, abort_flag)) { ok = false; break; }
          r_kv = false;
          const uint64_t vd = v_desc0 + static_cast<uint64_t>((2 * r * TILE) >> 4);
          const uint64_t kd_next = kv_desc0 + static_cast<uint64_t>(((2 * r + 1) * TILE) >> 4);   // K_{j+1}
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int n_i = i == 0 ? it.n0 : it.n1;
            if (j >= n_i) continue;
            uint32_t& cp = i == 0 ? cp0 : cp1;
            uint32_t& co = i == 0 ? co0 : co1;
            bool& r_h0 = i == 0 ? r_p00 : r_p10;
            bool& r_h1 = i == 0 ? r_p01 : r_p11;
            const uint32_t pj = cp & 1u;
            if (!r_h0 && !mbar_wait(&p_full[2 * i], pj, abort_flag)) { ok = false; break; }
            r_h0 = false;
            // the item's first PV overwrites the accumulator: the previous item's output must have been read
            if (j == 0 && co > 0 && !mbar_wait(&o_free[i], (co - 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_o = tmem_base + 256 + i * BN, a_p = tmem_base + i * BN;
            r_h1 = pv4_peek(d_o, a_p, vd, idesc_pv, j != 0 ? 1u : 0u, pf0 + (2 * i + 1) * 8, pj);
            if (!r_h1 && !mbar_wait(&p_full[2 * i + 1], pj, abort_flag)) { ok = false; break; }
            r_h1 = false;
            tc_fence_after();
            ++cp;
            // tested meanwhile: after tile 0 the first P half of tile 1 (this key block), after tile 1
            // the next ring entry and the first P half of tile 0 for the next key block of this item
            const uint32_t peek1 = i == 0 ? pf0 + 2 * 8 : kvf0 + ((g + 1) & 1u) * 8;
            const uint32_t par1 = i == 0 ? (cp1 & 1u) : (((g + 1) >> 1) & 1u);
            const uint32_t peek2 = pf0, par2 = cp0 & 1u;   // (used after tile 1 only: cp0 already counts this block)
            const uint64_t qd = q_desc0 + static_cast<uint64_t>((i * TILE) >> 4);
            bool t1, t2;
            if (j + 1 < n_i)
              pv4_s_commit_peek2<D, true>(d_o, a_p + 32, vd + 512, idesc_pv, tmem_base + i * BN, qd, kd_next, idesc_qk,
                                          sf0 + i * 8, peek1, par1, peek2, par2, t1, t2);
            else   // the tile's last key block of the item: the commit says that the output is complete
              pv4_s_commit_peek2<D, false>(d_o, a_p + 32, vd + 512, idesc_pv, tmem_base + i * BN, qd, kd_next, idesc_qk,
                                           of0 + i * 8, peek1, par1, peek2, par2, t1, t2);
            if (j + 1 == n_i) ++co;   // this tile's output of the item is complete behind that commit
            if (i == 0) {
              r_p10 = t1 && j < it.n1;
            } else {
              r_kv = t1 && j + 1 < it.nmax;
              r_p00 = t2 && j + 1 < it.n0;
            }
          }
          if (!ok) break;
          mma_commit(&kv_empty[r]);
          // the item's last QK^T (of the longer tile) has just been issued: Q and K_0 may be replaced when it is done
          if (j + 2 == it.nmax) mma_commit(q_empty);
        }
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit(drain_bar);
        mbar_wait(drain_bar, 0, &zero, 20000000ull);
      }
    }
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax / epilogue
    reg_alloc<V2P_REGS_SOFTMAX>();
    const int i = warp >> 2;                      // query tile of this warpgroup
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale_log2;
    const uint32_t s_addr = tmem_base + lane_base + i * BN;
    const uint32_t o_addr = tmem_base + lane_base + 256 + i * BN;
    uint32_t cs = 0;   // completions of s_full[i] consumed so far
    uint32_t cf = 0;   // completions of o_full[i] consumed so far
    int g0 = 0;        // ring entries used by the items before this one
    bool ok = true;
    for (int rd = 0; rd * static_cast<int>(gridDim.x) < items && ok; ++rd) {
      const int k = item_of_round(rd);
      if (k >= items) continue;
      const Item it = decode(k);
      const int n_mine = i == 0 ? it.n0 : it.n1;
      const int qi = it.q0 + i * BM + r;
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < n_mine; ++j, ++cs) {
        if (!mbar_wait(&s_full[i], cs & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int kv0 = j * BN;
        int limit = p.Skv - kv0;
        if (p.causal) limit = min(limit, qi + off + 1 - kv0);
        softmax_block<T, D>(s_addr, o_addr, j, limit, c, m, l, lane, [&](int half) { mbar_arrive(&p_full[2 * i + half]); });
      }
      if (!ok) break;
      // epilogue: the commit behind the tile's last PV
      if (n_mine > 0) {
        if (!mbar_wait(&o_full[i], cf & 1u, abort_flag)) { ok = false; break; }
        ++cf;
        tc_fence_after();
      }
      auto released = [&]() {   // the accumulator has been read: the next item's first PV may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[i]);
      };
      if (n_mine > 0) {
        // Staging space: the ring entry of the item's second-to-last key block (the one that will
        // next receive the following item's first K / V).  The longer tile's last block has left it
        // by the time either tile gets here, except that the shorter tile of a causal pair finishes
        // one block early and has to wait for the other tile to leave that block.
        const int G = g0 + it.nmax - 2;   // global index of that key block; negative: the entry was never used
        if (G >= 0 && !mbar_wait(&kv_empty[G & 1], (G >> 1) & 1u, abort_flag)) { ok = false; break; }
        uint8_t* stg = kv_smem + (2 * (G >= 0 ? (G & 1) : 1)) * TILE + warp * (32 * D * 2);
        store_output_tma<T, D>(p, o_addr, l, it.b, it.h, it.q0 + i * BM + quarter * 32, lane, stg, &tmO, released);
      } else {
        store_output_direct<T, D>(p, o_addr, false, l, it.b, it.h, it.q0 + i * BM + quarter * 32, lane, released);
      }
      if (it.nmax > 0) {
        if (lane == 0) mbar_arrive(stage_done);
        g0 += it.nmax;
      }
    }
    if (!ok && lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  } else {
    reg_dealloc<V2P_REGS_SERVICE>();   // warps 10-11: only the hand-over
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Grid size and dealing order of the persistent kernel.  Items are head-major; with a causal mask
// the pairs of a head cost from 3 to 4 * pairs - 1 key-block units, and what matters is the most
// loaded CTA.  Two schemes are compared on the item costs themselves: every SM with the snake order
// (balanced when the SM count is a multiple of the pairs per head and the number of rounds is
// even), or the largest grid coprime to the pairs per head with the plain order (every CTA meets
// all pair positions in turn).  Without a mask all items are equal and every SM is used.
struct PersistPlan { int grid; int snake; };
inline PersistPlan persist_plan(const FmhaParams& p, int items, int pairs, int sms) {
  if (items <= sms) return {items, 0};
  if (!p.causal) return {sms, 0};
  auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
  int g_plain = sms;
  while (g_plain > 1 && gcd(g_plain, pairs) != 1) --g_plain;
  const int off = p.Skv - p.Sq;
  auto cost = [&](int pos) {   // key blocks of both tiles of the pair at position `pos` of a head, plus a fixed part
    const int pr = pairs - 1 - pos;
    const int q0 = pr * 2 * BM;
    const int e0 = std::min(p.Skv, q0 + BM + off), e1 = std::min(p.Skv, q0 + 2 * BM + off);
    const int n0 = e0 > 0 ? (e0 + BN - 1) / BN : 0, n1 = e1 > 0 ? (e1 + BN - 1) / BN : 0;
    return n0 + n1 + 3;
  };
  std::vector<int> pos_cost(pairs);
  for (int i = 0; i < pairs; ++i) pos_cost[i] = cost(i);
  auto max_load = [&](int grid, int snake) {
    std::vector<int64_t> load(grid, 0);
    for (int k = 0; k < items; ++k) {
      const int r = k / grid;
      int c = k % grid;
      if (snake && (r & 1)) c = grid - 1 - c;
      load[c] += pos_cost[k % pairs];
    }
    int64_t m = 0;
    for (int64_t v : load) m = std::max(m, v);
    return m;
  };
  // the decision depends on (items, pairs, mask geometry) only: remember the last one per thread
  thread_local int key[4] = {-1, -1, -1, -1};
  thread_local PersistPlan last = {0, 0};
  if (key[0] == items && key[1] == pairs && key[2] == p.Sq && key[3] == p.Skv) return last;
  const int64_t a = max_load(sms, 1), b = max_load(g_plain, 0);
  last = a <= b ? PersistPlan{sms, 1} : PersistPlan{g_plain, 0};
  key[0] = items; key[1] = pairs; key[2] = p.Sq; key[3] = p.Skv;
  return last;
}

template <typename T, int D>
int launch_fmha2p(const CUtensorMap& tmO, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                  const FmhaParams& p, uint32_t fmt, cudaStream_t stream) {
  constexpr int DB = D / 64;
  constexpr int TILE = DB * TILE16K;
  constexpr int SMEM = 7 * TILE + 1024 + 256;
  auto kern = fmha_fwd_kernel2p<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "fmha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, BM, BN);
  const uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, BM, D);
  const int pairs = (p.q_tiles + 1) / 2;
  const int64_t items64 = static_cast<int64_t>(pairs) * p.B * p.H;
  if (items64 > INT32_MAX) return fail(KCG_ERR_UNSUPPORTED, "fmha: too many work items for the persistent kernel");
  const PersistPlan plan = persist_plan(p, static_cast<int>(items64), pairs, sm_count());
  launch_overlapped(kern, dim3(static_cast<unsigned>(plan.grid)), dim3(V2_THREADS), SMEM, stream, tmO, tmQ, tmK, tmV, p, idesc_qk,
                    idesc_pv, plan.snake);
  return check_launch("fmha_fwd_kernel2p");
}
