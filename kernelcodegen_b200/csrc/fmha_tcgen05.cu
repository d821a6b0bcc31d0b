// Fused multi-head attention forward for sm_100a.
//
// The reference fuses BatchedMatmul(Q,K^T) -> Softmax -> BatchedMatmul(P,V) into one
// flash-attention style kernel (src/Optimizer/Optimizer.cc:2606-2860): a CTA owns Br query
// rows, walks the keys in blocks of Bc, keeps running row max / row sum, and rescales the
// output accumulator, all in fp32 FFMA with the score tile staged through shared memory.
// This kernel keeps that blockwise online-softmax algorithm and moves both contractions to
// the tensor cores:
//   warp 0      TMA loads of the 128-row Q tile (once) and of 128-key K and V tiles into
//               2-stage rings;
//   warp 1      one thread issues tcgen05.mma: S = Q K^T into one of two score buffers in
//               tensor memory, then O += P V with V consumed straight from its row-major
//               [key, d] tile (an "MN-major" B operand), so no transpose is needed;
//   warps 2-5   softmax: one thread per query row reads its 128 scores from tensor memory
//               (a row never spans lanes, so the row max / row sum need no shuffles),
//               computes exp2 of the scaled scores, writes P as the 16-bit A operand of the
//               second MMA and, when the running max moved, rescales O in tensor memory.
// The score MMA of key block j+1 is issued before the PV MMA of block j, so tensor-core
// work overlaps the softmax of the previous block.
//
// Extensions over the reference (which has neither): a softmax scale folded into the
// exp2 argument, and a causal mask that also skips key blocks above the diagonal.
#include "common.cuh"
#include "tcgen05.cuh"

#include <algorithm>
#include <vector>


// Pairs of exponentials whose index has all bits of this mask set are computed on the FMA pipe
// (exp2_pair_fma) instead of the special-function unit: 0 none, 7 one in eight, 3 one in four.
// Measured on B8 H32 D128 (two-tile kernel): one in four gains 2.5 % at S = 1024 and on causal
// S = 2048 and 0.4 % at S = 4096, one in eight about half of that; accuracy is unchanged (2.3e-3).
#ifndef KCG_FMHA_EMU_MASK
#define KCG_FMHA_EMU_MASK 3
#endif

namespace kcg {

int* device_status_word();
int encode_tmap_sw128(CUtensorMap* out, int dtype, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box);

namespace {
using namespace sm100;

constexpr int BM = 128;          // query rows per CTA
constexpr int BN = 128;          // keys per block
constexpr int KV_STAGES = 2;
constexpr int TILE16K = 16384;   // one 128-row x 128-byte swizzled block
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units: rescale O only when the max grew by > 2^8

struct FmhaParams {
  void* O;
  int64_t o_sb, o_sh, o_ss;  // element strides of O
  int B, H, Sq, Skv;
  float scale_log2;          // softmax_scale * log2(e)
  int causal;
  int q_tiles;
  int* status;
  // further copies of O (same strides), typically this rank's slices inside the gather buffers
  // of peer GPUs; written by the two-tile kernel's epilogue
  void* extra_o[7];
  int n_extra;
  // or: the same block of O inside a multicast mapping of every rank's gather buffer (one store
  // per row segment, delivered to all ranks by NVSwitch, instead of O plus every extra_o)
  void* mc_o;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}


// ---- packed fp32x2 arithmetic (two lanes of fp32 in one 64-bit register) --------------------
// sm_100 executes fma / add on fp32 pairs in one instruction, which halves the FMA-pipe
// instruction count of the softmax.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// 2^x for a pair of values on the FMA and integer pipes instead of the special-function unit:
// n = round(x) by the magic-number addition, f = x - n in [-0.5, 0.5], 2^f by a cubic (relative
// error 1.1e-4, far below the rounding of a 16-bit P), and n added into the exponent field.
// Arguments below -126 (masked scores are -inf) give exactly 0, like the flushing ex2.approx.ftz.
__device__ __forceinline__ void exp2_pair_fma(uint64_t x2, float& p0, float& p1) {
  float x0, x1;
  f2_unpack(x2, x0, x1);
  const uint64_t xc = x2;
  const uint64_t magic = f2_pack(12582912.f, 12582912.f), nmagic = f2_pack(-12582912.f, -12582912.f);
  const uint64_t t = f2_add(xc, magic);                 // low mantissa bits = n
  const uint64_t n = f2_add(t, nmagic);                 // n as a float
  const uint64_t fr = f2_fma(n, f2_pack(-1.f, -1.f), xc);
  uint64_t p = f2_fma(fr, f2_pack(0.0555054f, 0.0555054f), f2_pack(0.2402265f, 0.2402265f));
  p = f2_fma(p, fr, f2_pack(0.6931472f, 0.6931472f));
  p = f2_fma(p, fr, f2_pack(1.0f, 1.0f));
  float t0, t1, q0, q1;
  f2_unpack(t, t0, t1);
  f2_unpack(p, q0, q1);
  p0 = x0 < -126.f ? 0.f : __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  p1 = x1 < -126.f ? 0.f : __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// kPTmem: P is written to tensor memory and the PV MMA reads its A operand from there;
// otherwise P goes through a swizzled shared-memory tile.
template <typename T, int D, bool kPTmem>
__global__ void __launch_bounds__(NUM_THREADS, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FmhaParams p, const uint32_t idesc_qk,
                const uint32_t idesc_pv) {
  constexpr int DB = D / 64;                 // 128-byte blocks along the head dimension
  constexpr int QK_TILE = DB * TILE16K;      // bytes of a Q, K or V tile
  constexpr int P_BYTES = 2 * TILE16K;
  constexpr uint32_t S_COL0 = 0, O_COL = 256, P_COL = 384;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + QK_TILE;
  uint8_t* v_smem = k_smem + KV_STAGES * QK_TILE;
  uint8_t* p_smem = v_smem + KV_STAGES * QK_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint64_t* drain_bar = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Causal: the last query tiles have the most key blocks; start them first.
  const int qt = p.causal ? (p.q_tiles - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qt * BM;
  const int off = p.Skv - p.Sq;  // key index of the diagonal for query 0
  int kv_end = p.Skv;
  if (p.causal) kv_end = min(p.Skv, q0 + BM + off);
  const int n_tiles = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      mbar_expect_tx(q_full, QK_TILE);
#pragma unroll
      for (int d = 0; d < DB; ++d) tma_load_4d(q_smem + d * TILE16K, &tmQ, q_full, d * 64, q0, h, b);
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t s = j % KV_STAGES, ph = (j / KV_STAGES) & 1u;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], QK_TILE);
#pragma unroll
        for (int d = 0; d < DB; ++d)
          tma_load_4d(k_smem + s * QK_TILE + d * TILE16K, &tmK, &k_full[s], d * 64, j * BN, h, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag)) { ok = false; issued = j; break; }
        mbar_expect_tx(&v_full[s], QK_TILE);
#pragma unroll
        for (int d = 0; d < DB; ++d)
          tma_load_4d(v_smem + s * QK_TILE + d * TILE16K, &tmV, &v_full[s], d * 64, j * BN, h, b);
        issued = j + 1;
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mbar_wait(q_full, 0, &zero, 2000000ull);
        for (int j = issued > KV_STAGES ? issued - KV_STAGES : 0; j < issued; ++j) {
          mbar_wait(&k_full[j % KV_STAGES], (j / KV_STAGES) & 1u, &zero, 2000000ull);
          mbar_wait(&v_full[j % KV_STAGES], (j / KV_STAGES) & 1u, &zero, 2000000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    bool ok = n_tiles > 0;
    const uint32_t q_addr = smem_u32(q_smem);
    const uint32_t p_addr = smem_u32(p_smem);
    auto issue_s = [&](int j) -> bool {
      const uint32_t s = j % KV_STAGES, ph = (j / KV_STAGES) & 1u;
      const uint32_t sb = j & 1u, sph = (j >> 1) & 1u;
      if (!mbar_wait(&k_full[s], ph, abort_flag)) return false;
      if (!mbar_wait(&s_empty[sb], sph ^ 1u, abort_flag)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(k_smem + s * QK_TILE);
#pragma unroll
        for (int d = 0; d < DB; ++d)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss<Kind::F16>(tmem_base + S_COL0 + sb * BN,
                              make_smem_desc(q_addr + d * TILE16K + k * 32, 16, 1024),
                              make_smem_desc(k_addr + d * TILE16K + k * 32, 16, 1024), idesc_qk,
                              (d | k) != 0 ? 1u : 0u);
        mma_commit(&k_empty[s]);
        mma_commit(&s_full[sb]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = mbar_wait(q_full, 0, abort_flag);
    if (ok) ok = issue_s(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
      const uint32_t s = j % KV_STAGES, ph = (j / KV_STAGES) & 1u;
      if (!mbar_wait(&v_full[s], ph, abort_flag)) { ok = false; break; }
      if (!mbar_wait(p_full, j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(v_smem + s * QK_TILE);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t bdesc = make_smem_desc(v_addr + kk * 2048, TILE16K, 1024);
          const uint32_t accumulate = (j | kk) != 0 ? 1u : 0u;
          if constexpr (kPTmem) {
            mma_ts_f16(tmem_base + O_COL, tmem_base + P_COL + kk * 8, bdesc, idesc_pv, accumulate);
          } else {
            const uint64_t adesc = make_smem_desc(p_addr + (kk >> 2) * TILE16K + (kk & 3) * 32, 16, 1024);
            mma_ss<Kind::F16>(tmem_base + O_COL, adesc, bdesc, idesc_pv, accumulate);
          }
        }
        mma_commit(&v_empty[s]);
        mma_commit(pv_done);
      }
      __syncwarp();
    }
    if (!ok && n_tiles > 0) {
      if (lane == 0) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mma_commit(drain_bar);
        mbar_wait(drain_bar, 0, &zero, 20000000ull);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;            // row within the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + r;                        // global query index
    const float c = p.scale_log2;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t sb = j & 1u, sph = (j >> 1) & 1u;
      if (!mbar_wait(&s_full[sb], sph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_base + S_COL0 + sb * BN;
      const int kv0 = j * BN;
      // Columns >= limit are masked: beyond the keys, or above the causal diagonal.
      int limit = p.Skv - kv0;
      if (p.causal) limit = min(limit, qi + off + 1 - kv0);
      const bool need_mask = limit < BN;
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        uint32_t sreg[32];
        tmem_ld32(s_addr + cc * 32, sreg);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (cc * 32 + i < limit) mx = fmaxf(mx, __uint_as_float(sreg[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sreg[i]));
        }
      }
      const float mt = mx * c;
      float alpha = 1.f;
      bool rescale = false;
      if (mt > m + kRescaleThreshold || m == -INFINITY) {
        if (mt > m) {
          alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - mt);
          rescale = (j > 0);
          m = mt;
        }
      }
      const float m_eff = (m == -INFINITY) ? 0.f : m;
      // pass 2: p = exp2(s*c - m), packed to 16 bits, row sum in fp32
      uint32_t pk[BN / 2];
      float lsum = 0.f;
#pragma unroll
      for (int cc = 0; cc < BN / 32; ++cc) {
        uint32_t sreg[32];
        tmem_ld32(s_addr + cc * 32, sreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(sreg[i]), c, -m_eff));
          float p1 = fast_exp2(fmaf(__uint_as_float(sreg[i + 1]), c, -m_eff));
          if (need_mask) {
            if (cc * 32 + i >= limit) p0 = 0.f;
            if (cc * 32 + i + 1 >= limit) p1 = 0.f;
          }
          lsum += p0 + p1;
          pk[cc * 16 + i / 2] = pack2<T>(p0, p1);
        }
      }
      // S(j) is fully read: hand the score buffer back to the MMA warp.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      // P buffer and O are free once the PV MMA of the previous block has finished.
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
          const float a = rescale ? alpha : 1.f;
#pragma unroll 1
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t oreg[32];
            tmem_ld32(tmem_base + lane_base + O_COL + cc * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * a);
            tmem_st32(tmem_base + lane_base + O_COL + cc * 32, oreg);
          }
          tmem_wait_st();
        }
      }
      l = l * alpha + lsum;
      if constexpr (kPTmem) {
        tmem_st32(tmem_base + lane_base + P_COL, reinterpret_cast<uint32_t(&)[32]>(pk[0]));
        tmem_st32(tmem_base + lane_base + P_COL + 32, reinterpret_cast<uint32_t(&)[32]>(pk[32]));
        tmem_wait_st();
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          uint8_t* dst = p_smem + (q >> 3) * TILE16K + r * 128 + (((q & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // epilogue: O / l -> global
    if (ok && n_tiles > 0) ok = mbar_wait(pv_done, (n_tiles - 1) & 1u, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.0f / l : 0.f;
      T* orow = static_cast<T*>(p.O) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh +
                static_cast<int64_t>(qi) * p.o_ss;
#pragma unroll 1
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t oreg[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem_base + lane_base + O_COL + cc * 32, oreg);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = 0u;
        }
        if (qi < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
            o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
            o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
            o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = o;
          }
        }
      }
    } else if (lane == 0 && !*abort_flag) {
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

// One key block of the online softmax for the calling thread's query row.  The 128 scores of the
// row sit in tensor memory at s_addr (this thread's lane); columns >= limit are masked.  On return
// P (16-bit, 64 columns) has replaced the first half of the scores, handed to the MMA thread in
// two halves through arrive(half) (called by lane 0 after the warp's stores are complete), the
// output accumulator at o_addr has been rescaled if the running maximum m moved by more than the
// threshold, and m and the running row sum l are up to date.  All 32 lanes of the warp call it.
struct NoHook {
  __device__ __forceinline__ bool operator()() const { return true; }
};

// Two optional hooks serve the kernel whose warpgroups take alternate key blocks of one tile:
// decided() is called (by all lanes) as soon as this block's value of m is final — before the
// exponentials on the ordinary path — and wait_o() before the accumulator is touched for a rescale
// (it returns false if its wait timed out; the rescale is then skipped and the caller gives up).
template <typename T, int D, typename Arrive, typename Decided = NoHook, typename WaitO = NoHook>
__device__ __forceinline__ bool softmax_block(uint32_t s_addr, uint32_t o_addr, int j, int limit, float c, float& m,
                                              float& l, int lane, Arrive arrive, Decided decided = Decided(),
                                              WaitO wait_o = WaitO()) {
  bool hooks_ok = true;
  uint32_t sreg[BN];
  tmem_ld64(s_addr, reinterpret_cast<uint32_t(&)[64]>(sreg[0]));
  tmem_ld64(s_addr + 64, reinterpret_cast<uint32_t(&)[64]>(sreg[64]));
  tmem_wait_ld();
  if (limit < BN) {
#pragma unroll
    for (int k = 0; k < BN; ++k)
      if (k >= limit) sreg[k] = 0xff800000u;  // -inf
  }
  // eight independent chains of 3-input max (8 dependent steps instead of 16)
  float mx[8];
#pragma unroll
  for (int a = 0; a < 8; ++a) mx[a] = fmaxf(__uint_as_float(sreg[2 * a]), __uint_as_float(sreg[2 * a + 1]));
#pragma unroll
  for (int k = 16; k < BN; k += 16) {
#pragma unroll
    for (int a = 0; a < 8; ++a) mx[a] = max3(mx[a], __uint_as_float(sreg[k + 2 * a]), __uint_as_float(sreg[k + 2 * a + 1]));
  }
  const float mt = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * c;
  uint64_t lsum_a = 0ull, lsum_b = 0ull;  // two (+0.f, +0.f) accumulators
  const uint64_t c2 = f2_pack(c, c);
  // exponentials of one half of the row (64 scores -> 32 packed words, written in place over
  // the words already consumed), then the hand-over of that half of P to the MMA thread
  auto exp_half = [&](int half, uint64_t nm2) {
#pragma unroll
    for (int k = half * 64; k < half * 64 + 64; k += 2) {
      const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sreg[k]), __uint_as_float(sreg[k + 1])), c2, nm2);
      float p0, p1;
      if (KCG_FMHA_EMU_MASK != 0 && ((k >> 1) & KCG_FMHA_EMU_MASK) == KCG_FMHA_EMU_MASK) {
        exp2_pair_fma(x2, p0, p1);
      } else {
        float x0, x1;
        f2_unpack(x2, x0, x1);
        p0 = fast_exp2(x0);
        p1 = fast_exp2(x1);
      }
      if ((k >> 1) & 1) lsum_b = f2_add(lsum_b, f2_pack(p0, p1));
      else lsum_a = f2_add(lsum_a, f2_pack(p0, p1));
      sreg[k >> 1] = pack2<T>(p0, p1);  // in place: word k/2 is never read again
    }
  };
  auto hand_over = [&](int half) {
    tmem_st32(s_addr + half * 32, reinterpret_cast<uint32_t(&)[32]>(sreg[half * 32]));
    tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) arrive(half);
  };
  float alpha = 1.f;
  bool half0_done = false;
  // Speculative path (every block after the first that needs no mask): the exponentials of the
  // first half start at once with the running maximum m, so that the maximum of this block is
  // computed in the shadow of the special-function unit instead of in front of it.  That is
  // exact whenever the block's maximum stays within the rescale threshold of m, which is the
  // condition under which m would have been kept anyway; otherwise (rare once a few blocks have
  // been seen) the first half is read again from tensor memory and redone on the ordinary path.
  const bool speculate = __all_sync(0xffffffffu, j > 0 && limit >= BN && m != -INFINITY);
  if (speculate) {
    const float neg_m0 = -m;
    exp_half(0, f2_pack(neg_m0, neg_m0));
    if (!__any_sync(0xffffffffu, mt > m + kRescaleThreshold)) {
      decided();
      hand_over(0);
      half0_done = true;
    } else {
      tmem_ld64(s_addr, reinterpret_cast<uint32_t(&)[64]>(sreg[0]));   // the first 32 words were overwritten
      tmem_wait_ld();
      lsum_a = 0ull;
      lsum_b = 0ull;
    }
  }
  if (!half0_done) {
    bool rescale = false;
    if ((mt > m + kRescaleThreshold || m == -INFINITY) && mt > m) {
      alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - mt);
      rescale = (j > 0);
      m = mt;
    }
    // In the two-tile kernels S_i(j) being complete means PV_i(j-1) is complete, so O_i may be
    // rescaled at once; a kernel where that does not hold passes wait_o.
    if (__any_sync(0xffffffffu, rescale)) {
      hooks_ok = wait_o();
      if (hooks_ok) {
        tc_fence_after();
        const float a = rescale ? alpha : 1.f;
#pragma unroll 1
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t oreg[32];
          tmem_ld32(o_addr + cc * 32, oreg);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) oreg[k] = __float_as_uint(__uint_as_float(oreg[k]) * a);
          tmem_st32(o_addr + cc * 32, oreg);
        }
      }
    }
    decided();
    const float neg_m = (m == -INFINITY) ? 0.f : -m;
    exp_half(0, f2_pack(neg_m, neg_m));
    hand_over(0);
  }
  {
    const float neg_m = (m == -INFINITY) ? 0.f : -m;
    exp_half(1, f2_pack(neg_m, neg_m));
    hand_over(1);
  }
  float l0, l1;
  f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
  l = l * alpha + (l0 + l1);
  return hooks_ok;
}

// The key-block step for the kernel that keeps P in tensor-memory columns of its own (p_addr, 64
// columns) instead of over the scores.  The score row then leaves tensor memory for good as soon
// as it has been read — release_s() is called by lane 0 right after the load — so the MMA thread
// may refill the score buffer while this block's exponentials run.  The row's scores stay in
// registers for the whole step (P is packed into a separate 32-word buffer per half), so the
// speculative path can redo a half without reading tensor memory again.  decided() is called by
// all lanes once this block's value of m is final; wait_o() before the accumulator is touched for
// a rescale and wait_p() before P(j) overwrites the P written two blocks earlier (both return
// false if their wait timed out); arrive() by lane 0 when all 64 columns of P are in place.
template <typename T, int D, typename ReleaseS, typename Decided, typename WaitO, typename WaitP, typename Arrive>
__device__ __forceinline__ bool softmax_block_px(uint32_t s_addr, uint32_t o_addr, uint32_t p_addr, int j, int limit,
                                                 float c, float& m, float& l, int lane, ReleaseS release_s,
                                                 Decided decided, WaitO wait_o, WaitP wait_p, Arrive arrive) {
  uint32_t sreg[BN];
  tmem_ld64(s_addr, reinterpret_cast<uint32_t(&)[64]>(sreg[0]));
  tmem_ld64(s_addr + 64, reinterpret_cast<uint32_t(&)[64]>(sreg[64]));
  tmem_wait_ld();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) release_s();
  if (limit < BN) {
#pragma unroll
    for (int k = 0; k < BN; ++k)
      if (k >= limit) sreg[k] = 0xff800000u;  // -inf
  }
  float mx[8];
#pragma unroll
  for (int a = 0; a < 8; ++a) mx[a] = fmaxf(__uint_as_float(sreg[2 * a]), __uint_as_float(sreg[2 * a + 1]));
#pragma unroll
  for (int k = 16; k < BN; k += 16) {
#pragma unroll
    for (int a = 0; a < 8; ++a) mx[a] = max3(mx[a], __uint_as_float(sreg[k + 2 * a]), __uint_as_float(sreg[k + 2 * a + 1]));
  }
  const float mt = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * c;
  uint64_t lsum_a = 0ull, lsum_b = 0ull;
  const uint64_t c2 = f2_pack(c, c);
  // P of the first half goes to a buffer of its own (that half may have to be redone from the
  // scores); P of the second half overwrites the first half's scores, which are dead by then.  The
  // registers a tcgen05.st reads are not touched again before tcgen05.wait::st.
  uint32_t pk[32];
  auto exp_half = [&](int half, uint64_t nm2, uint32_t* dst) {
#pragma unroll
    for (int k = half * 64; k < half * 64 + 64; k += 2) {
      const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sreg[k]), __uint_as_float(sreg[k + 1])), c2, nm2);
      float p0, p1;
      if (KCG_FMHA_EMU_MASK != 0 && ((k >> 1) & KCG_FMHA_EMU_MASK) == KCG_FMHA_EMU_MASK) {
        exp2_pair_fma(x2, p0, p1);
      } else {
        float x0, x1;
        f2_unpack(x2, x0, x1);
        p0 = fast_exp2(x0);
        p1 = fast_exp2(x1);
      }
      if ((k >> 1) & 1) lsum_b = f2_add(lsum_b, f2_pack(p0, p1));
      else lsum_a = f2_add(lsum_a, f2_pack(p0, p1));
      dst[(k >> 1) & 31] = pack2<T>(p0, p1);
    }
  };
  float alpha = 1.f;
  bool half0_done = false, ok = true;
  const bool speculate = __all_sync(0xffffffffu, j > 0 && limit >= BN && m != -INFINITY);
  if (speculate) {   // exponentials first, the block's maximum in their shadow (see softmax_block)
    const float neg_m0 = -m;
    exp_half(0, f2_pack(neg_m0, neg_m0), pk);
    if (!__any_sync(0xffffffffu, mt > m + kRescaleThreshold)) {
      decided();
      ok = wait_p();
      tmem_st32(p_addr, pk);
      half0_done = true;
    } else {
      lsum_a = 0ull;   // the scores are still in registers: redo the half on the ordinary path
      lsum_b = 0ull;
    }
  }
  if (!half0_done) {
    bool rescale = false;
    if ((mt > m + kRescaleThreshold || m == -INFINITY) && mt > m) {
      alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - mt);
      rescale = (j > 0);
      m = mt;
    }
    if (__any_sync(0xffffffffu, rescale)) {
      ok = wait_o();
      if (ok) {
        tc_fence_after();
        const float a = rescale ? alpha : 1.f;
#pragma unroll 1
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t oreg[32];
          tmem_ld32(o_addr + cc * 32, oreg);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) oreg[k] = __float_as_uint(__uint_as_float(oreg[k]) * a);
          tmem_st32(o_addr + cc * 32, oreg);
        }
      }
    }
    decided();
    const float neg_m = (m == -INFINITY) ? 0.f : -m;
    exp_half(0, f2_pack(neg_m, neg_m), pk);
    ok = wait_p() && ok;
    tmem_st32(p_addr, pk);
  }
  {
    const float neg_m = (m == -INFINITY) ? 0.f : -m;
    exp_half(1, f2_pack(neg_m, neg_m), sreg);
    tmem_st32(p_addr + 32, reinterpret_cast<uint32_t(&)[32]>(sreg[0]));
  }
  tmem_wait_st();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) arrive();
  float l0, l1;
  f2_unpack(f2_add(lsum_a, lsum_b), l0, l1);
  l = l * alpha + (l0 + l1);
  return ok;
}

// Stores the calling thread's finished output row: O / l, rounded to T.  With extra outputs
// (copies of O in other GPUs' memory) the warp's 32 rows are staged through `stg` (32 rows x D
// elements of shared memory that is idle by now) and leave as whole rows to every destination.
//
// With a tensor map of O (tmO, the two-tile kernel) and no extra outputs, the rows of a tile
// that had key blocks leave through the copy engine instead: the warp packs them into swizzled
// boxes of 32 rows x 128 bytes in `stg` and one lane issues a TMA store per box, which writes
// whole lines and clips at Sq.  Stored directly, every warp instruction touches 32 different
// lines with 16 bytes each.
template <typename T, int D>
__device__ __forceinline__ void store_output(const FmhaParams& p, uint32_t o_addr, bool have_o, float l, int b, int h,
                                             int row0, int lane, uint8_t* stg, int peer_seed,
                                             const CUtensorMap* tmO = nullptr) {
  const int qi = row0 + lane;   // this thread's query row; row0 is the first row of the warp
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;
  if (tmO != nullptr && have_o && p.n_extra == 0 && p.mc_o == nullptr) {
    if (row0 >= p.Sq) return;
#pragma unroll 1
    for (int cc = 0; cc < D / 32; ++cc) {
      uint32_t oreg[32];
      tmem_ld32(o_addr + cc * 32, oreg);
      tmem_wait_ld();
      uint8_t* box = stg + (cc >> 1) * 4096 + lane * 128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
        o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
        o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
        o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
        const int gc = (cc & 1) * 4 + g;   // 16-byte chunk within the box's 128-byte row
        *reinterpret_cast<uint4*>(box + ((gc ^ (lane & 7)) << 4)) = o;
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int d = 0; d < D / 64; ++d) tma_store_4d(tmO, stg + d * 4096, d * 64, row0, h, b);
      tma_store_commit();
      tma_store_wait_read<0>();   // the CTA's shared memory must outlive the copy engine's reads
    }
    return;
  }
  T* orow = static_cast<T*>(p.O) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh +
            static_cast<int64_t>(qi) * p.o_ss;
  if (p.n_extra > 0 || p.mc_o != nullptr) {
    // Staged stores for remote destinations: this warp's 32 output rows pass through idle shared
    // memory, swizzled, and leave as whole rows of D elements (256 bytes at D = 128), so that a
    // store to another GPU's memory carries full lines; every destination receives the same registers.
    constexpr int ROWB = D * 2;          // bytes per output row
    constexpr int CH = ROWB / 16;        // 16-byte chunks per row
    constexpr int RPI = 32 / CH;         // rows per store instruction
#pragma unroll 1
    for (int cc = 0; cc < D / 32; ++cc) {
      uint32_t oreg[32];
      if (have_o) {
        tmem_ld32(o_addr + cc * 32, oreg);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) oreg[k] = 0u;
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
        o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
        o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
        o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
        const int gc = cc * 4 + g;
        *reinterpret_cast<uint4*>(stg + lane * ROWB + ((gc ^ (lane & (CH - 1))) << 4)) = o;
      }
    }
    __syncwarp();
    const int64_t slice = static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh;
#pragma unroll
    for (int it = 0; it < 32 / RPI; ++it) {
      const int rr = it * RPI + lane / CH, ch = lane % CH;
      const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * ROWB + ((ch ^ (rr & (CH - 1))) << 4));
      if (row0 + rr < p.Sq) {
        const int64_t off = slice + static_cast<int64_t>(row0 + rr) * p.o_ss + ch * 8;
        if (p.mc_o != nullptr) {
          multimem_st16(static_cast<T*>(p.mc_o) + off, v);
          continue;
        }
        *reinterpret_cast<uint4*>(static_cast<T*>(p.O) + off) = v;
        // peers in an order that differs from CTA to CTA and from step to step, so that the
        // stores of the whole grid do not queue up on one NVLink destination at a time
        const int peer0 = p.n_extra > 0 ? static_cast<int>(static_cast<unsigned>(peer_seed + it) % static_cast<unsigned>(p.n_extra)) : 0;
        for (int e = 0; e < p.n_extra; ++e) {
          const int d = (e + peer0) % p.n_extra;
          *reinterpret_cast<uint4*>(static_cast<T*>(p.extra_o[d]) + off) = v;
        }
      }
    }
  } else {
#pragma unroll 1
    for (int cc = 0; cc < D / 32; ++cc) {
      uint32_t oreg[32];
      if (have_o) {
        tmem_ld32(o_addr + cc * 32, oreg);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) oreg[k] = 0u;
      }
      if (qi < p.Sq) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
          o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
          o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
          o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = o;
        }
      }
    }
  }
}

// The calling thread's finished output row, read out of tensor memory in one go and stored straight
// from registers (no shared memory).  `released` runs as soon as the accumulator has been read, before
// the conversion and the stores: the persistent kernel lets the next item's first PV overwrite it then.
template <typename T, int D, typename Released>
__device__ __forceinline__ void store_output_direct(const FmhaParams& p, uint32_t o_addr, bool have_o, float l, int b, int h,
                                                    int row0, int lane, Released released) {
  const int qi = row0 + lane;
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;
  T* orow = static_cast<T*>(p.O) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh +
            static_cast<int64_t>(qi) * p.o_ss;
  uint32_t oreg[D];
  if (have_o) {
#pragma unroll
    for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(o_addr + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[cc * 32]));
    tmem_wait_ld();
    released();
  } else {
#pragma unroll
    for (int k = 0; k < D; ++k) oreg[k] = 0u;
  }
  if (qi < p.Sq) {
#pragma unroll
    for (int g = 0; g < D / 8; ++g) {
      uint4 o;
      o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
      o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
      o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
      o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
      *reinterpret_cast<uint4*>(orow + g * 8) = o;
    }
  }
}

// The warp's 32 finished output rows through the copy engine: read out of tensor memory in one go
// (`released` runs right after, the accumulator may be overwritten from then on), packed into
// swizzled boxes of 32 rows x 128 bytes in `stg` (D * 64 bytes of shared memory nobody else uses
// at this moment) and handed to TMA stores, which write whole lines and clip at Sq.  Returns when
// the copy engine has read the staging tile.
template <typename T, int D, typename Released>
__device__ __forceinline__ void store_output_tma(const FmhaParams& p, uint32_t o_addr, float l, int b, int h, int row0,
                                                 int lane, uint8_t* stg, const CUtensorMap* tmO, Released released) {
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;
  uint32_t oreg[D];
#pragma unroll
  for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(o_addr + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&oreg[cc * 32]));
  tmem_wait_ld();
  released();
  if (row0 >= p.Sq) return;
#pragma unroll
  for (int g = 0; g < D / 8; ++g) {
    uint4 o;
    o.x = pack2<T>(__uint_as_float(oreg[g * 8 + 0]) * inv_l, __uint_as_float(oreg[g * 8 + 1]) * inv_l);
    o.y = pack2<T>(__uint_as_float(oreg[g * 8 + 2]) * inv_l, __uint_as_float(oreg[g * 8 + 3]) * inv_l);
    o.z = pack2<T>(__uint_as_float(oreg[g * 8 + 4]) * inv_l, __uint_as_float(oreg[g * 8 + 5]) * inv_l);
    o.w = pack2<T>(__uint_as_float(oreg[g * 8 + 6]) * inv_l, __uint_as_float(oreg[g * 8 + 7]) * inv_l);
    // box g / 8 (64 columns = 128 bytes per row), 16-byte chunk g % 8 within the row
    *reinterpret_cast<uint4*>(stg + (g >> 3) * 4096 + lane * 128 + (((g & 7) ^ (lane & 7)) << 4)) = o;
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < D / 64; ++d) tma_store_4d(tmO, stg + d * 4096, d * 64, row0, h, b);
    tma_store_commit();
    tma_store_wait_read<0>();
  }
  __syncwarp();
}

// ---- MMA groups of the two-tile kernel's issuing thread ------------------------------------
// The issuing thread is one of the kernel's two bottlenecks: an MMA of 128x128x16 takes the thread
// about as long to issue (65-75 clocks) as the tensor pipe needs to run it (68), and a barrier
// test needs ~140 clocks to answer.  Tested on its own in front of a batch of MMAs, every barrier
// would idle the pipe for that long, five times per key block.  So each batch is one asm block
// that first issues a non-blocking test of the barrier(s) needed *after* it, then the MMAs (and
// the commit), and reads the answers last; only a barrier that was not complete yet is waited
// for in the ordinary way.
//
// Four PV k-steps: O (+)= P[:, 16 kk .. 16 kk + 16) V[16 kk .., :], kk = kk0 .. kk0 + 3.  a_p / vd address
// k-step kk0 (P advances 8 tensor-memory columns, the V descriptor 2048 bytes per k-step).
__device__ __forceinline__ bool pv4_peek(uint32_t d_o, uint32_t a_p, uint64_t vd, uint32_t idesc, uint32_t acc_first,
                                         uint32_t peek_bar, uint32_t peek_par) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P, Q, T;\n\t.reg .b32 a1, a2, a3;\n\t.reg .b64 v1, v2, v3;\n\t"
      "setp.ne.b32 P, %5, 0;\n\t"
      "setp.eq.b32 T, %5, %5;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 Q, [%6], %7;\n\t"
      "add.u32 a1, %2, 8;\n\tadd.u32 a2, %2, 16;\n\tadd.u32 a3, %2, 24;\n\t"
      "add.s64 v1, %3, 128;\n\tadd.s64 v2, %3, 256;\n\tadd.s64 v3, %3, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, P;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], v1, %4, T;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], v2, %4, T;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], v3, %4, T;\n\t"
      "selp.u32 %0, 1, 0, Q;\n\t}"
      : "=r"(ok)
      : "r"(d_o), "r"(a_p), "l"(vd), "r"(idesc), "r"(acc_first), "r"(peek_bar), "r"(peek_par)
      : "memory");
  return ok != 0;
}
// Four PV k-steps (always accumulating), then — if kWithS — the next score tile S = Q K^T (D / 16
// k-steps, the first one overwriting), then the commit on `commit_bar`; two barriers are tested.
// qd / kd: descriptors of k-step 0 (k-steps advance 32 bytes, the second 64-element half of the
// head dimension lies one 16 KB block further).
#define KCG_SS_STEP(OFF, PRED)                                                            \
  "add.s64 qx, %7, " #OFF ";\n\tadd.s64 kx, %8, " #OFF ";\n\t"                             \
  "tcgen05.mma.cta_group::1.kind::f16 [%6], qx, kx, %9, " #PRED ";\n\t"
template <int D, bool kWithS>
__device__ __forceinline__ void pv4_s_commit_peek2(uint32_t d_o, uint32_t a_p, uint64_t vd, uint32_t idesc_pv, uint32_t d_s,
                                                   uint64_t qd, uint64_t kd, uint32_t idesc_qk, uint32_t commit_bar,
                                                   uint32_t peek1, uint32_t par1, uint32_t peek2, uint32_t par2,
                                                   bool& ok1, bool& ok2) {
  uint32_t r1, r2;
#define KCG_PV4                                                                                    \
  "{\n\t.reg .pred F, Q1, Q2, T;\n\t.reg .b32 a1, a2, a3;\n\t.reg .b64 v1, v2, v3, qx, kx;\n\t"     \
  "setp.eq.b32 T, %2, %2;\n\t"                                                                     \
  "setp.ne.b32 F, %2, %2;\n\t"                                                                     \
  "mbarrier.test_wait.parity.shared::cta.b64 Q1, [%11], %12;\n\t"                                  \
  "mbarrier.test_wait.parity.shared::cta.b64 Q2, [%13], %14;\n\t"                                  \
  "add.u32 a1, %3, 8;\n\tadd.u32 a2, %3, 16;\n\tadd.u32 a3, %3, 24;\n\t"                           \
  "add.s64 v1, %4, 128;\n\tadd.s64 v2, %4, 256;\n\tadd.s64 v3, %4, 384;\n\t"                       \
  "tcgen05.mma.cta_group::1.kind::f16 [%2], [%3], %4, %5, T;\n\t"                                  \
  "tcgen05.mma.cta_group::1.kind::f16 [%2], [a1], v1, %5, T;\n\t"                                  \
  "tcgen05.mma.cta_group::1.kind::f16 [%2], [a2], v2, %5, T;\n\t"                                  \
  "tcgen05.mma.cta_group::1.kind::f16 [%2], [a3], v3, %5, T;\n\t"
#define KCG_TAIL                                                                                   \
  "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%10];\n\t"               \
  "selp.u32 %0, 1, 0, Q1;\n\tselp.u32 %1, 1, 0, Q2;\n\t}"
#define KCG_OPERANDS                                                                               \
  : "=r"(r1), "=r"(r2)                                                                             \
  : "r"(d_o), "r"(a_p), "l"(vd), "r"(idesc_pv), "r"(d_s), "l"(qd), "l"(kd), "r"(idesc_qk),         \
    "r"(commit_bar), "r"(peek1), "r"(par1), "r"(peek2), "r"(par2)                                  \
  : "memory"
  if constexpr (!kWithS) {
    asm volatile(KCG_PV4 KCG_TAIL KCG_OPERANDS);
  } else if constexpr (D == 128) {
    asm volatile(KCG_PV4 KCG_SS_STEP(0, F) KCG_SS_STEP(2, T) KCG_SS_STEP(4, T) KCG_SS_STEP(6, T) KCG_SS_STEP(1024, T)
                     KCG_SS_STEP(1026, T) KCG_SS_STEP(1028, T) KCG_SS_STEP(1030, T) KCG_TAIL KCG_OPERANDS);
  } else {
    asm volatile(KCG_PV4 KCG_SS_STEP(0, F) KCG_SS_STEP(2, T) KCG_SS_STEP(4, T) KCG_SS_STEP(6, T) KCG_TAIL KCG_OPERANDS);
  }
#undef KCG_PV4
#undef KCG_TAIL
#undef KCG_OPERANDS
  ok1 = r1 != 0;
  ok2 = r2 != 0;
}
#undef KCG_SS_STEP

// ---------------------------------------------------------------------------------------------
// Version 2: two 128-query tiles per CTA.
//
//   warps 0-3   softmax warpgroup of query tile 0 (one thread per row, TMEM lanes 0-127)
//   warps 4-7   softmax warpgroup of query tile 1
//   warp 8      TMA loader: both Q tiles and K_0 once, then (V_j, K_{j+1}) per key block
//   warp 9      MMA issuer
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).
// P_i (16-bit, 64 columns) overwrites the first half of S_i once the owning thread has read
// its score row.  The MMA thread issues, per key block j and tile i:  O_i += P_i(j) V_j  and
// right behind it  S_i(j+1) = Q_i K_{j+1}^T.  MMAs of one thread execute in issue order, so
// S_i(j+1) cannot overwrite P_i(j) before it has been read, and when the softmax threads see
// S_i(j+1) complete, O_i is stable (PV_i(j) is behind them) and may be rescaled.  While tile
// i is in its softmax, the tensor pipe works on tile 1-i, and every K / V tile is loaded once
// for 256 query rows.
// 12 warps: two softmax warpgroups, then a warpgroup holding the loader (warp 8) and the MMA
// issuer (warp 9); warps 10-11 only take part in the register hand-over.  The third warpgroup
// gives most of its registers to the softmax warpgroups (setmaxnreg), whose 128-element score
// rows otherwise spill at the 168 registers a 384-thread CTA gets per thread.
constexpr int V2_THREADS = 384;
constexpr int V2_REGS_SOFTMAX = 208, V2_REGS_SERVICE = 88;   // 2*128*208 + 128*88 = 64512 = 384 x 168, what the CTA is launched with
static_assert(2 * 128 * V2_REGS_SOFTMAX + 128 * V2_REGS_SERVICE <= V2_THREADS * 168, "register split exceeds the CTA's allocation");

template <typename T, int D, int NSLOT>
__global__ void __launch_bounds__(V2_THREADS, 1)
fmha_fwd_kernel2(const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FmhaParams p, const uint32_t idesc_qk,
                 const uint32_t idesc_pv) {
  constexpr int DB = D / 64;
  constexpr int TILE = DB * TILE16K;   // bytes of one Q, K or V tile

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* q_smem = smem;                   // [2][TILE]
  uint8_t* kv_smem = smem + 2 * TILE;       // [NSLOT][TILE]
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_smem + NSLOT * TILE);
  uint64_t* q_full = bars;                  // [1]
  uint64_t* kv_full = bars + 1;             // [NSLOT]
  uint64_t* kv_empty = kv_full + NSLOT;     // [NSLOT]
  uint64_t* s_full = kv_empty + NSLOT;      // [2]
  uint64_t* p_full = s_full + 2;            // [2 tiles][2 column halves]
  uint64_t* drain_bar = p_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = (p.q_tiles + 1) / 2;
  const int pr = p.causal ? (pairs - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = pr * 2 * BM;
  const int off = p.Skv - p.Sq;
  // key blocks of the two tiles, as scalars: an array indexed by the tile would live in local memory
  const int kv_end0 = p.causal ? min(p.Skv, q0 + BM + off) : p.Skv;
  const int kv_end1 = p.causal ? min(p.Skv, q0 + 2 * BM + off) : p.Skv;
  const int n_blk0 = kv_end0 > 0 ? (kv_end0 + BN - 1) / BN : 0;
  const int n_blk1 = kv_end1 > 0 ? (kv_end1 + BN - 1) / BN : 0;
  const int n_max = max(n_blk0, n_blk1);  // == n_blk1: the later rows see at least as many keys

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
    mbar_init(q_full, 1);
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 4);
      mbar_init(&p_full[2 * i + 1], 4);
    }
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
    reg_dealloc<V2_REGS_SERVICE>();
    if (lane == 0 && n_max > 0) {
      bool ok = true;
      // Ring layout: K_0 travels with the Q tiles (slot 4, never reused); afterwards one ring
      // entry per key block j holds V_j (slot 2r) and K_{j+1} (slot 2r+1), r = j & 1, under a
      // single full / empty barrier pair, so the MMA thread pays one wait and one commit per block.
      mbar_expect_tx(q_full, 3 * TILE);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int d = 0; d < DB; ++d)
          tma_load_4d(q_smem + i * TILE + d * TILE16K, &tmQ, q_full, d * 64, q0 + i * BM, h, b);
#pragma unroll
      for (int d = 0; d < DB; ++d) tma_load_4d(kv_smem + 4 * TILE + d * TILE16K, &tmK, q_full, d * 64, 0, h, b);
      int j = 0;
      for (; j < n_max; ++j) {
        const uint32_t r = j & 1u, ph = (j >> 1) & 1u;
        if (!mbar_wait(&kv_empty[r], ph ^ 1u, abort_flag)) { ok = false; break; }
        const bool more = j + 1 < n_max;
        mbar_expect_tx(&kv_full[r], more ? 2 * TILE : TILE);
#pragma unroll
        for (int d = 0; d < DB; ++d)
          tma_load_4d(kv_smem + (2 * r) * TILE + d * TILE16K, &tmV, &kv_full[r], d * 64, j * BN, h, b);
        if (more) {
#pragma unroll
          for (int d = 0; d < DB; ++d)
            tma_load_4d(kv_smem + (2 * r + 1) * TILE + d * TILE16K, &tmK, &kv_full[r], d * 64, (j + 1) * BN, h, b);
        }
      }
      if (!ok) {
        if (!*abort_flag) { *abort_flag = 1; *p.status = KCG_ERR_TIMEOUT; __threadfence_system(); }
        int zero = 0;
        mbar_wait(q_full, 0, &zero, 2000000ull);
        for (int u = j > 2 ? j - 2 : 0; u < j; ++u) mbar_wait(&kv_full[u & 1], (u >> 1) & 1u, &zero, 2000000ull);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    reg_dealloc<V2_REGS_SERVICE>();
    bool ok = n_max > 0;
    const uint32_t q_addr = smem_u32(q_smem);
    // Shared-memory descriptors are built once; an MMA's descriptor is a base plus a constant in
    // the address field (16-byte units; the sums stay inside the 14-bit field), so that nothing
    // but an add sits between two MMAs of a batch.
    const uint64_t q_desc0 = make_smem_desc(q_addr, 16, 1024);
    const uint64_t kv_desc0 = make_smem_desc(smem_u32(kv_smem), 16, 1024);          // K tiles (K-major)
    const uint64_t v_desc0 = make_smem_desc(smem_u32(kv_smem), TILE16K, 1024);      // V tiles (MN-major)
    auto issue_s = [&](int i, int j) {  // S_i(j) = Q_i K_j^T   (lane 0 only)
      const uint64_t qd = q_desc0 + static_cast<uint64_t>((i * TILE) >> 4);
      const uint64_t kd = kv_desc0 + static_cast<uint64_t>(((j == 0 ? 4 : 2 * ((j - 1) & 1) + 1) * TILE) >> 4);
#pragma unroll
      for (int d = 0; d < DB; ++d)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss<Kind::F16>(tmem_base + i * BN, qd + ((d * TILE16K + k * 32) >> 4), kd + ((d * TILE16K + k * 32) >> 4),
                            idesc_qk, (d | k) != 0 ? 1u : 0u);
    };
    // One thread runs the whole issue loop: nothing here needs the other lanes, and a single
    // thread has no reconvergence points between a barrier wait and the MMAs that follow it.
    // (An MMA is accepted only when the tensor pipe has room, so issuing blocks for about as
    // long as the MMAs run: every instruction between two MMAs is tensor-pipe idle time.)
    if (lane == 0 && ok) {
      ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if ((i == 0 ? n_blk0 : n_blk1) > 0) {
            issue_s(i, 0);
            mma_commit(&s_full[i]);
          }
      }
      // Barriers already seen complete by a test that rode along with an earlier MMA batch
      bool r_kv = false, r_p00 = false, r_p01 = false, r_p10 = false, r_p11 = false;
      const uint32_t kvf0 = smem_u32(kv_full), pf0 = smem_u32(p_full), sf0 = smem_u32(s_full);
      for (int j = 0; j < n_max && ok; ++j) {
        if (!r_kv && !mbar_wait(&kv_full[j & 1], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
        r_kv = false;
        const uint32_t pj = j & 1u;
        const uint64_t vd = v_desc0 + static_cast<uint64_t>((2 * (j & 1) * TILE) >> 4);
        const uint64_t kd_next = kv_desc0 + static_cast<uint64_t>(((2 * (j & 1) + 1) * TILE) >> 4);   // K_{j+1}
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int n_i = i == 0 ? n_blk0 : n_blk1;
          if (j >= n_i) continue;
          bool& r_h0 = i == 0 ? r_p00 : r_p10;
          bool& r_h1 = i == 0 ? r_p01 : r_p11;
          // P arrives in two column halves; the first four k-steps of PV start on the first
          if (!r_h0 && !mbar_wait(&p_full[2 * i], pj, abort_flag)) { ok = false; break; }
          r_h0 = false;
          tc_fence_after();
          const uint32_t d_o = tmem_base + 256 + i * BN, a_p = tmem_base + i * BN;
          r_h1 = pv4_peek(d_o, a_p, vd, idesc_pv, j != 0 ? 1u : 0u, pf0 + (2 * i + 1) * 8, pj);
          if (!r_h1 && !mbar_wait(&p_full[2 * i + 1], pj, abort_flag)) { ok = false; break; }
          r_h1 = false;
          tc_fence_after();
          // Second half of PV, the next score tile behind it, one commit for both (the next score
          // tile, or the finished output, is ready); tested meanwhile: what the thread needs next —
          // after tile 0 the first P half of tile 1, after tile 1 the next K/V ring entry and the
          // first P half of tile 0 for the next key block.
          const uint32_t peek1 = i == 0 ? pf0 + 2 * 8 : kvf0 + ((j + 1) & 1) * 8;
          const uint32_t par1 = i == 0 ? pj : static_cast<uint32_t>(((j + 1) >> 1) & 1);
          const uint32_t peek2 = pf0, par2 = pj ^ 1u;   // p_full[0] of key block j + 1 (used after tile 1 only)
          const uint64_t qd = q_desc0 + static_cast<uint64_t>((i * TILE) >> 4);
          bool t1, t2;
          if (j + 1 < n_i)
            pv4_s_commit_peek2<D, true>(d_o, a_p + 32, vd + 512, idesc_pv, tmem_base + i * BN, qd, kd_next, idesc_qk,
                                        sf0 + i * 8, peek1, par1, peek2, par2, t1, t2);
          else
            pv4_s_commit_peek2<D, false>(d_o, a_p + 32, vd + 512, idesc_pv, tmem_base + i * BN, qd, kd_next, idesc_qk,
                                         sf0 + i * 8, peek1, par1, peek2, par2, t1, t2);
          if (i == 0) {
            r_p10 = t1 && j < n_blk1;
          } else {
            r_kv = t1 && j + 1 < n_max;
            r_p00 = t2 && j + 1 < n_blk0;
          }
        }
        if (ok) mma_commit(&kv_empty[j & 1]);
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
    reg_alloc<V2_REGS_SOFTMAX>();
    const int i = warp >> 2;                      // query tile of this warpgroup
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + i * BM + r;
    const float c = p.scale_log2;
    const int n_mine = i == 0 ? n_blk0 : n_blk1;
    const uint32_t s_addr = tmem_base + lane_base + i * BN;
    const uint32_t o_addr = tmem_base + lane_base + 256 + i * BN;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait(&s_full[i], j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BN;
      int limit = p.Skv - kv0;
      if (p.causal) limit = min(limit, qi + off + 1 - kv0);
      softmax_block<T, D>(s_addr, o_addr, j, limit, c, m, l, lane, [&](int half) { mbar_arrive(&p_full[2 * i + half]); });
    }
    // epilogue: the commit after the last PV arrives on s_full once more
    if (ok && n_mine > 0) ok = mbar_wait(&s_full[i], n_mine & 1u, abort_flag);
    if (ok) {
      tc_fence_after();
      store_output<T, D>(p, o_addr, n_mine > 0, l, b, h, q0 + i * BM + quarter * 32, lane,
                         q_smem + i * TILE + quarter * (32 * D * 2),
                         static_cast<int>(blockIdx.x + blockIdx.y) + warp, &tmO);
    } else if (lane == 0 && !*abort_flag) {
      *abort_flag = 1;
      *p.status = KCG_ERR_TIMEOUT;
      __threadfence_system();
    }
  } else {
    reg_dealloc<V2_REGS_SERVICE>();   // warps 10-11: only the hand-over
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

#include "fmha_pair_kernel.cuh"
#include "fmha_split_kernel.cuh"
#include "fmha_persist_kernel.cuh"

template <typename T, int D>
int launch_fmha2(const CUtensorMap& tmO, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FmhaParams& p,
                 uint32_t fmt, cudaStream_t stream) {
  constexpr int DB = D / 64;
  constexpr int TILE = DB * TILE16K;
  constexpr int NSLOT = 5;  // two (V, K) ring entries plus the slot of K_0
  constexpr int SMEM = (2 + NSLOT) * TILE + 1024 + 256;
  auto kern = fmha_fwd_kernel2<T, D, NSLOT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "fmha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, BM, BN);
  const uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, BM, D);
  dim3 grid((p.q_tiles + 1) / 2, p.B * p.H);
  launch_overlapped(kern, grid, dim3(V2_THREADS), SMEM, stream, tmO, tmQ, tmK, tmV, p, idesc_qk, idesc_pv);
  return check_launch("fmha_fwd_kernel2");
}

template <typename T, int D, bool kPTmem>
int launch_fmha(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FmhaParams& p,
                uint32_t fmt, cudaStream_t stream) {
  constexpr int DB = D / 64;
  constexpr int SMEM = DB * TILE16K * (1 + 2 * KV_STAGES) + 2 * TILE16K + 1024 + 256;
  auto kern = fmha_fwd_kernel<T, D, kPTmem>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "fmha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, BM, BN);
  const uint32_t idesc_pv = make_idesc(fmt, fmt, 0, 1, BM, D);
  dim3 grid(p.q_tiles, p.B * p.H);
  kern<<<grid, NUM_THREADS, SMEM, stream>>>(tmQ, tmK, tmV, p, idesc_qk, idesc_pv);
  return check_launch("fmha_fwd_kernel");
}

thread_local int g_p_in_tmem = -1;  // per calling thread; -1: choose by shape

}  // namespace

// Kernel variant: -1 (default) picks by shape; 0 / 1 = one query tile per CTA with P through
// shared / tensor memory; 2 = two query tiles per CTA; 3 = a CTA pair on four query tiles; 4 = a
// CTA pair with one tile per CTA whose warpgroups take alternate key blocks.
extern "C" __attribute__((visibility("default"))) void kcg_fmha_set_p_in_tmem(int v) { g_p_in_tmem = v; }

}  // namespace kcg

namespace kcg {
namespace {
int fmha_fwd_impl(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D, float softmax_scale, int causal,
                  const void* Q, const int64_t q_strides[3], const void* K, const int64_t k_strides[3], const void* V,
                  const int64_t v_strides[3], void* O, const int64_t o_strides[3], void* stream, void* const* extra_o,
                  int n_extra, void* mc_o = nullptr);
}
}  // namespace kcg

extern "C" int kcg_fmha_fwd(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                            float softmax_scale, int causal, const void* Q, const int64_t q_strides[3],
                            const void* K, const int64_t k_strides[3], const void* V,
                            const int64_t v_strides[3], void* O, const int64_t o_strides[3], void* stream) {
  kcg::clear_error();
  return kcg::fmha_fwd_impl(dtype, B, H, Sq, Skv, D, softmax_scale, causal, Q, q_strides, K, k_strides, V, v_strides, O,
                            o_strides, stream, nullptr, 0);
}

// Attention forward whose epilogue also performs the all-gather of O: the slices this rank
// computes are stored into every rank's gathered tensor, peers included, as whole output rows.
extern "C" int kcg_fmha_fwd_allgather(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                                      float softmax_scale, int causal, const void* Q, const int64_t q_strides[3],
                                      const void* K, const int64_t k_strides[3], const void* V,
                                      const int64_t v_strides[3], void* const* gathered, int world, int rank,
                                      int64_t batch_offset, const int64_t o_strides[3], void* stream) {
  using namespace kcg;
  clear_error();
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(KCG_ERR_INVALID_ARG, "fmha_allgather: world %d (1..8), rank %d", world, rank);
  if (!gathered || !o_strides || batch_offset < 0) return fail(KCG_ERR_INVALID_ARG, "fmha_allgather: bad argument");
  void* mine = nullptr;
  void* others[8];
  int n_others = 0;
  for (int r = 0; r < world; ++r) {
    if (!gathered[r]) return fail(KCG_ERR_INVALID_ARG, "fmha_allgather: gathered[%d] is null", r);
    void* blk = static_cast<char*>(gathered[r]) + static_cast<size_t>(batch_offset) * o_strides[0] * 2;
    if (r == rank) mine = blk; else others[n_others++] = blk;
  }
  return fmha_fwd_impl(dtype, B, H, Sq, Skv, D, softmax_scale, causal, Q, q_strides, K, k_strides, V, v_strides, mine,
                       o_strides, stream, others, n_others);
}

// The same with the gather done by NVSwitch: every output row is stored once, to the multicast
// address of its place in the gathered tensor, and arrives in every rank's buffer.
extern "C" int kcg_fmha_fwd_allgather_multicast(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D,
                                                float softmax_scale, int causal, const void* Q,
                                                const int64_t q_strides[3], const void* K, const int64_t k_strides[3],
                                                const void* V, const int64_t v_strides[3], void* gathered_local,
                                                void* gathered_multicast, int64_t batch_offset,
                                                const int64_t o_strides[3], void* stream) {
  using namespace kcg;
  clear_error();
  if (!gathered_local || !gathered_multicast || !o_strides || batch_offset < 0)
    return fail(KCG_ERR_INVALID_ARG, "fmha_allgather_multicast: bad argument");
  const size_t shift = static_cast<size_t>(batch_offset) * o_strides[0] * 2;
  return fmha_fwd_impl(dtype, B, H, Sq, Skv, D, softmax_scale, causal, Q, q_strides, K, k_strides, V, v_strides,
                       static_cast<char*>(gathered_local) + shift, o_strides, stream, nullptr, 0,
                       static_cast<char*>(gathered_multicast) + shift);
}

namespace kcg {
namespace {
int fmha_fwd_impl(int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D, float softmax_scale, int causal,
                  const void* Q, const int64_t q_strides[3], const void* K, const int64_t k_strides[3], const void* V,
                  const int64_t v_strides[3], void* O, const int64_t o_strides[3], void* stream, void* const* extra_o,
                  int n_extra, void* mc_o) {
  if (B < 0 || H < 0 || Sq < 0 || Skv < 0) return fail(KCG_ERR_INVALID_ARG, "fmha: negative extent");
  if (dtype != KCG_BF16 && dtype != KCG_F16)
    return fail(KCG_ERR_UNSUPPORTED, "fmha: dtype %d has no kernel (bfloat16, float16)", dtype);
  if (D != 64 && D != 128) return fail(KCG_ERR_UNSUPPORTED, "fmha: head dimension %lld (64 or 128)", static_cast<long long>(D));
  if (B == 0 || H == 0 || Sq == 0) return KCG_OK;
  if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides)
    return fail(KCG_ERR_INVALID_ARG, "fmha: null pointer");
  if (Skv == 0) return fail(KCG_ERR_INVALID_ARG, "fmha: Skv must be positive");
  if (B * H > 65535 || Sq > INT32_MAX || Skv > INT32_MAX)
    return fail(KCG_ERR_UNSUPPORTED, "fmha: batch*heads above 65535 is not supported");
  const void* ptrs[4] = {Q, K, V, O};
  const int64_t* strides[4] = {q_strides, k_strides, v_strides, o_strides};
  for (int t = 0; t < 4; ++t) {
    if (!aligned16(ptrs[t])) return fail(KCG_ERR_ALIGNMENT, "fmha: tensor %d is not 16-byte aligned", t);
    for (int i = 0; i < 3; ++i)
      if (strides[t][i] % 8 != 0 || strides[t][i] <= 0)
        return fail(KCG_ERR_ALIGNMENT, "fmha: strides must be positive multiples of 8 elements (tensor %d stride %d = %lld)",
                    t, i, static_cast<long long>(strides[t][i]));
  }
  CUtensorMap tm[5];   // Q, K, V with 128-row boxes; K again with 64-row boxes (the CTA-pair kernel's halves); O, 32-row boxes
  const int64_t seq[5] = {Sq, Skv, Skv, Skv, Sq};
  const int src[5] = {0, 1, 2, 1, 3};
  for (int t = 0; t < 5; ++t) {
    uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(seq[t]), static_cast<uint64_t>(H),
                        static_cast<uint64_t>(B)};
    uint64_t st[3] = {static_cast<uint64_t>(strides[src[t]][2]) * 2, static_cast<uint64_t>(strides[src[t]][1]) * 2,
                      static_cast<uint64_t>(strides[src[t]][0]) * 2};
    uint32_t box[4] = {64, t == 3 ? 64u : (t == 4 ? 32u : 128u), 1, 1};
    int rc = encode_tmap_sw128(&tm[t], dtype, ptrs[src[t]], 4, dims, st, box);
    if (rc) return rc;
  }
  FmhaParams p;
  p.O = O; p.o_sb = o_strides[0]; p.o_sh = o_strides[1]; p.o_ss = o_strides[2];
  p.B = static_cast<int>(B); p.H = static_cast<int>(H); p.Sq = static_cast<int>(Sq); p.Skv = static_cast<int>(Skv);
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.q_tiles = static_cast<int>((Sq + BM - 1) / BM);
  p.status = device_status_word();
  if (!p.status) return fail(KCG_ERR_CUDA, "fmha: could not allocate the host-mapped status word");
  p.n_extra = n_extra;
  p.mc_o = mc_o;
  if (mc_o && !aligned16(mc_o)) return fail(KCG_ERR_ALIGNMENT, "fmha: the multicast output address is not 16-byte aligned");
  for (int i = 0; i < 7; ++i) p.extra_o[i] = i < n_extra ? extra_o[i] : nullptr;
  for (int i = 0; i < n_extra; ++i)
    if (!extra_o[i] || !aligned16(extra_o[i])) return fail(KCG_ERR_ALIGNMENT, "fmha: extra output %d is null or not 16-byte aligned", i);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t fmt = dtype == KCG_BF16 ? 1u : 0u;
  // By shape: the persistent two-tile kernel when there is more than one tile of queries, else one
  // tile per CTA.  (The CTA-pair kernels, variants 3 and 4, are correct on every test shape but
  // measured slower; they and the one-shot two-tile kernel stay selectable.)  Extra outputs (the
  // gather epilogues) are written by variants 2 and 3.
  int variant = g_p_in_tmem >= 0 ? g_p_in_tmem : (Sq > BM ? 5 : 1);
  if ((variant == 3 || variant == 4) && D != 128) variant = 2;
  if ((n_extra > 0 || mc_o) && (variant < 2 || variant >= 4)) variant = 2;
  if (variant == 5 && Sq <= BM) variant = 1;
  if (variant == 5) {
    if (dtype == KCG_BF16)
      return D == 128 ? launch_fmha2p<__nv_bfloat16, 128>(tm[4], tm[0], tm[1], tm[2], p, fmt, s)
                      : launch_fmha2p<__nv_bfloat16, 64>(tm[4], tm[0], tm[1], tm[2], p, fmt, s);
    return D == 128 ? launch_fmha2p<__half, 128>(tm[4], tm[0], tm[1], tm[2], p, fmt, s)
                    : launch_fmha2p<__half, 64>(tm[4], tm[0], tm[1], tm[2], p, fmt, s);
  }
  if (variant == 4)
    return dtype == KCG_BF16 ? launch_fmha_split<__nv_bfloat16>(tm[0], tm[3], tm[2], p, fmt, s)
                             : launch_fmha_split<__half>(tm[0], tm[3], tm[2], p, fmt, s);
  if (variant == 3)
    return dtype == KCG_BF16 ? launch_fmha_pair<__nv_bfloat16>(tm[0], tm[3], tm[2], p, fmt, s)
                             : launch_fmha_pair<__half>(tm[0], tm[3], tm[2], p, fmt, s);
#define KCG_FMHA(TT, DD)                                                                      \
  (variant == 2   ? launch_fmha2<TT, DD>(tm[4], tm[0], tm[1], tm[2], p, fmt, s)               \
   : variant == 1 ? launch_fmha<TT, DD, true>(tm[0], tm[1], tm[2], p, fmt, s)                 \
                  : launch_fmha<TT, DD, false>(tm[0], tm[1], tm[2], p, fmt, s))
  if (dtype == KCG_BF16) return D == 128 ? KCG_FMHA(__nv_bfloat16, 128) : KCG_FMHA(__nv_bfloat16, 64);
  return D == 128 ? KCG_FMHA(__half, 128) : KCG_FMHA(__half, 64);
#undef KCG_FMHA
}
}  // namespace
}  // namespace kcg
