// Flash-attention forward for sm_100a: O = softmax(Q K^T * sm_scale [+ causal mask]) V and the
// base-2 log-sum-exp of the scaled scores per query row.
//
// One CTA handles 256 query rows of one (batch, head) as two groups of 128; KV is walked in
// blocks of 128. Roles (384 threads):
//   warp 0       TMA loads: Q0, Q1 once per tile; K(j), V(j) through a 4-deep ring.
//   warp 1       one thread issues every tcgen05.mma, in the fixed order
//                QK0(0) QK1(0) | PV0(j) QK0(j+1) PV1(j) QK1(j+1) | ...   so that while one group's
//                softmax runs the tensor pipe works for the other group. PV_g(j) goes out in four
//                slices as the softmax publishes P in 32-column chunks, overlapping its tail.
//                (Measured alternatives that lost: one issuing thread per group, 715 vs 900
//                TFLOP/s - MMAs of two streams interleave one by one; a Cody-Waite + cubic exp2
//                on the FMA pipe for 25-50 % of the elements, 5-20 % slower - issue-bound; and one
//                ex2.approx.ftz.bf16x2 per pair of scores - half the special-function instructions, P
//                produced directly in its stored precision - 983 vs 1106 TFLOP/s.)
//                S_g = Q_g K^T : SS MMA, 128 x 128 x D.    O_g += P_g V : TS MMA, P read from TMEM,
//                V is the MN-major B operand straight from its row-major tile.
//   warps 4-7    softmax + correction + epilogue for group 0;  warps 8-11 the same for group 1.
//                Thread t owns query row t of its group: tcgen05.ld 32x32b hands it whole rows, so
//                row max / row sum need no shuffles. Online softmax in the exp2 domain; the
//                accumulator is rescaled only when the running max grew by more than 2^8 (any lane
//                of the warp), otherwise the stale max stays the reference point and the final
//                O / l is unchanged. P (bf16) is written over the first half of S's columns.
// Tensor memory (512 columns): S0 | S1 | O0 | O1 with P_g aliasing S_g.
// Head dim 256 (a 128-row tile is 64 KB, an output accumulator 256 columns): the same kernel with one query group per
// CTA - Q | a two-deep K / V ring in shared memory, S0 | O0 in tensor memory, the second softmax warpgroup idle; the
// softmax of a block then runs with the tensor pipe idle, which weighs less here because a block carries twice the
// MMA work per score (measured 905 / 920 TFLOP/s at [4, 16, 8192, 256] non-causal / causal).
// In-order execution of one thread's tcgen05.mma stream gives the S/P write-after-read order
// (QK_g(j+1) is issued after PV_g(j)) and makes PV_g(j-1) complete before S_g(j) is signalled, so
// only the last PV of a tile carries a completion barrier of its own. The issuing thread probes
// the barrier it needs next (mbarrier.test_wait) before each batch of MMAs: a blocking wait costs
// it ~70 cycles even when the phase is complete, a probe issued ahead of the MMAs costs nothing.
//
// Counterpart in the reference: _attn_fwd_ws / _attn_fwd_ws_kernel,
// third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py:600-1249 (softmax :223-322,
// MMA order :413-597, correction :816-914, LSE :886-894), host entry `attention` :3491.
#include <string.h>

#include "attention_common.cuh"
#include "common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int ATT_THREADS = 384;
static constexpr int ATT_BM = 128;   // query rows per group
static constexpr int ATT_BN = 128;   // kv rows per block
static constexpr int ATT_KV_STAGES = 4;
static constexpr float ATT_RESCALE_THRESHOLD = 8.0f;
#ifndef ATT_PV_SLICES
#define ATT_PV_SLICES 4  // PV_g is issued in this many slices as P is published
#endif

struct AttnParams {
  CUtensorMap tmq, tmk, tmv;  // 3-D (D, S, B*H), box (64, 128, 1), 128-byte swizzle
  void* o;
  float* lse;
  int* status;
  int bh, s_q, s_kv;
  int q_tiles;  // ceil(s_q / 256)
  int units;    // q_tiles * bh
  int causal;
  int out_f16;
  float scale_log2;  // sm_scale * log2(e)
};

// G = query groups per CTA: 2 (256 query rows, the groups' MMAs and softmax passes interleaved), or 1 for head dim 256,
// where a tile is 64 KB and tensor memory holds one 128 x 256 output besides the scores: one group, a two-deep K / V ring.
template <int D, int G>
struct AttnSmem {
  static constexpr int TILE_BYTES = 128 * D * 2;  // one 128-row tile of Q, K or V
  static constexpr int KV_STAGES = G == 2 ? ATT_KV_STAGES : 2;
  static constexpr int Q_OFFSET = 0;
  static constexpr int KV_OFFSET = G * TILE_BYTES;
  static constexpr int BAR_OFFSET = KV_OFFSET + KV_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 4 + 2 * ATT_KV_STAGES + 14;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
};

struct AttnTile {
  int bh, q0, nkv;
  int nkv0;  // KV blocks the first 128-row group needs: one fewer than nkv when the last block lies wholly above its diagonal
};

// Heaviest tiles first (largest query block = most KV blocks under a causal mask), all heads of one query
// block before the next block. This order re-reads each head's K / V from HBM for every query tile (15.8 GB
// per launch at [4, 32, 8192, 128], 4 TB/s); head-major and L2-sized head-group orders cut that to ~1 GB but
// measured equal (non-causal) or 5-30 % slower (causal: the long tiles no longer start first), so it stays.
// Measured again with groups of heads sized to 16 / 32 MB of K + V, alternating with this order in one process
// (five rounds): [4, 32, 8192, 128] 999 / 992 against 1044 TFLOP/s non-causal and 930 / 931 against 967 causal;
// [32, 32, 1024, 128] 901 / 917 against 890 and 596 / 585 against 609.
template <int G>
__device__ __forceinline__ AttnTile attn_tile(const AttnParams& p, int unit) {
  AttnTile t;
  const int qb = p.q_tiles - 1 - unit / p.bh;
  t.bh = unit % p.bh;
  t.q0 = qb * G * ATT_BM;
  int nkv = (p.s_kv + ATT_BN - 1) / ATT_BN;
  t.nkv0 = nkv;
  if (p.causal) {
    t.nkv0 = min(nkv, (t.q0 + ATT_BM + ATT_BN - 1) / ATT_BN);
    nkv = min(nkv, (t.q0 + G * ATT_BM + ATT_BN - 1) / ATT_BN);
  }
  t.nkv = nkv;
  return t;
}

template <int D, bool F16, int G>
__global__ void __launch_bounds__(ATT_THREADS, 1) attention_fwd_kernel(const __grid_constant__ AttnParams p) {
  using L = AttnSmem<D, G>;
  constexpr bool TWO = G == 2;
  constexpr int KV_STAGES = L::KV_STAGES;
  constexpr int DBOX = D / 64;                 // 64-column TMA boxes per tile
  constexpr int BOX_BYTES = 128 * 128;         // 128 rows x 128 bytes
  constexpr uint32_t S_COLS = 128;
  constexpr uint32_t O_COL0 = 2 * S_COLS;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* q_full = bars;                      // [2]
  uint64_t* q_empty = bars + 2;                 // [2]
  uint64_t* kv_full = bars + 4;                 // [KV]
  uint64_t* kv_empty = kv_full + ATT_KV_STAGES; // [KV]
  uint64_t* s_full = kv_empty + ATT_KV_STAGES;  // [2] MMA -> softmax: S_g ready
  uint64_t* p_full = s_full + 2;                // [2][4] softmax -> MMA: 32-column chunk c of P_g written (128 arrivals)
  uint64_t* pv_done = p_full + 8;               // [2] MMA -> softmax: last PV_g of the tile complete
  uint64_t* o_free = pv_done + 2;               // [2] softmax -> MMA: O_g read out (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmq);
    tma_prefetch_desc(&p.tmk);
    tma_prefetch_desc(&p.tmv);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&s_full[i], 1);
      for (int c = 0; c < 4; ++c) mbar_init(&p_full[i * 4 + c], 128);
      mbar_init(&pv_done[i], 1);
      mbar_init(&o_free[i], 128);
    }
    for (int i = 0; i < ATT_KV_STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  int* const status = p.status;
  const int units = p.units;
  const uint32_t smem_a = smem_u32(smem);

  // Register re-partition: the load / MMA warpgroup needs few registers, the softmax warpgroups hold
  // a whole 128-column score row per thread.
  // (each role branch starts with its own setmaxnreg so that the instruction dominates the code it
  // governs; the four warps of the first warpgroup all execute the same decrease)
  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    reg_dealloc<104>();
    if (lane == 0) {
      const uint64_t pol_q = policy_evict_first();
      const uint64_t pol_kv = policy_evict_last();
      uint32_t kvs = 0, kvph = 0, tcount = 0;
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint64_t* bar, int row, int bh, uint64_t pol) {
        mbar_expect_tx(bar, L::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DBOX; ++b)
          tma_load_3d(smem + (dst - smem_a) + b * BOX_BYTES, tm, bar, b * 64, row, bh, pol);
      };
      auto load_kv = [&](const CUtensorMap* tm, int row, int bh) -> bool {
        if (!mbar_wait(&kv_empty[kvs], kvph ^ 1, status, WAIT_SMEM_EMPTY)) return false;
        load_tile(tm, smem_a + L::KV_OFFSET + kvs * L::TILE_BYTES, &kv_full[kvs], row, bh, pol_kv);
        if (++kvs == KV_STAGES) {
          kvs = 0;
          kvph ^= 1;
        }
        return true;
      };
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
        const AttnTile t = attn_tile<G>(p, unit);
        const uint32_t qph = (tcount & 1) ^ 1;
        if (!mbar_wait(&q_empty[0], qph, status, WAIT_SMEM_EMPTY)) break;
        load_tile(&p.tmq, smem_a + L::Q_OFFSET, &q_full[0], t.q0, t.bh, pol_q);
        if (!load_kv(&p.tmk, 0, t.bh)) break;
        if constexpr (TWO) {
          if (!mbar_wait(&q_empty[1], qph, status, WAIT_SMEM_EMPTY)) break;
          load_tile(&p.tmq, smem_a + L::Q_OFFSET + L::TILE_BYTES, &q_full[1], t.q0 + ATT_BM, t.bh, pol_q);
        }
        if (!load_kv(&p.tmv, 0, t.bh)) break;
        for (int j = 1; j < t.nkv && ok; ++j) {
          ok = load_kv(&p.tmk, j * ATT_BN, t.bh) && load_kv(&p.tmv, j * ATT_BN, t.bh);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    reg_dealloc<104>();
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc(1u, 1u, 0u, 0u, ATT_BM, ATT_BN);  // bf16 x bf16, both K-major
      const uint32_t idesc_pv = make_idesc(1u, 1u, 0u, 1u, ATT_BM, D);       // B (= V) MN-major
      constexpr uint32_t fmt_fix = F16 ? ((1u << 7) | (1u << 10)) : 0u;     // fp16: operand format 0
      const uint32_t idq = idesc_qk & ~fmt_fix, idp = idesc_pv & ~fmt_fix;
      const uint64_t qdesc0 = make_smem_desc(smem_a + L::Q_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t kdesc0 = make_smem_desc(smem_a + L::KV_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t vdesc0 = make_smem_desc(smem_a + L::KV_OFFSET, BOX_BYTES, 1024, SWIZZLE_128B);
      uint32_t kvs = 0, kvph = 0;  // ring position of the next unconsumed KV tile
      uint32_t it0 = 0, it1 = 0;   // kv iterations issued so far per group (phase source for the s / p barriers)
      uint32_t tcount = 0;
      bool ok = true;

      auto issue_qk = [&](int g, uint32_t kstage) {
        const uint64_t qd = qdesc0 + (uint64_t)((g * L::TILE_BYTES) >> 4);
        const uint64_t kd = kdesc0 + (uint64_t)((kstage * L::TILE_BYTES) >> 4);
        const uint32_t d_s = tmem_base + g * S_COLS;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = (uint64_t)(((k >> 2) * BOX_BYTES + (k & 3) * 32) >> 4);
          umma_f16_ss(d_s, qd + off, kd + off, idq, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[g]);
      };
      // PV_g in four slices: slice c (two MMAs, 32 kv rows) goes out as soon as the softmax has
      // published chunk c of P_g, so the MMA overlaps the tail of the softmax
      auto issue_pv = [&](int g, uint32_t vstage, uint32_t accum, uint32_t iph, bool ready, bool last) -> bool {
        const uint64_t vd = vdesc0 + (uint64_t)((vstage * L::TILE_BYTES) >> 4);
        const uint32_t d_o = tmem_base + O_COL0 + g * D;
        const uint32_t a_p = tmem_base + g * S_COLS;
#pragma unroll
        for (int c = 0; c < ATT_PV_SLICES; ++c) {
          // the softmax publishes P in four 32-column chunks; a slice waits for its last chunk (a
          // thread arrives on the chunk barriers in order)
          constexpr int CH = 4 / ATT_PV_SLICES;
          if (!ready && !mbar_wait(&p_full[g * 4 + c * CH + CH - 1], iph, status, WAIT_ATTN)) return false;
          tc_fence_after_sync();
          if (c + 1 < ATT_PV_SLICES)
            ready = mbar_test(&p_full[g * 4 + (c + 1) * CH + CH - 1], iph);  // probe ahead of this slice's MMAs
#pragma unroll
          for (int k = 2 * CH * c; k < 2 * CH * (c + 1); ++k)
            umma_f16_ts(d_o, a_p + k * 8, vd + (uint64_t)((k * 16 * 128) >> 4), idp, (k > 0) ? 1u : accum);
        }
        // S_g(j+1) is committed after this in the same in-order stream, so only the last PV of a
        // tile needs a completion signal of its own (the epilogue waits for it)
        if (last) umma_commit(&pv_done[g]);
        return true;
      };
      auto advance = [&]() {
        if (++kvs == KV_STAGES) {
          kvs = 0;
          kvph ^= 1;
        }
      };

      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
        const AttnTile t = attn_tile<G>(p, unit);
        const uint32_t tph = tcount & 1;
        // prologue: S_g(0) = Q_g K(0)^T
        uint32_t kcur = kvs, kcur_ph = kvph;
        advance();
        if (!mbar_wait(&q_full[0], tph, status, WAIT_ATTN)) break;
        if (!mbar_wait(&kv_full[kcur], kcur_ph, status, WAIT_SMEM_FULL)) break;
        tc_fence_after_sync();
        issue_qk(0, kcur);
        if constexpr (TWO) {
          if (!mbar_wait(&q_full[1], tph, status, WAIT_ATTN)) break;
          tc_fence_after_sync();
          issue_qk(1, kcur);
        }
        umma_commit(&kv_empty[kcur]);
        // Under a causal mask the last KV block of a tile can lie wholly above the first group's diagonal: that group
        // then runs one block fewer (n0 = n1 - 1) and the last iteration serves the second group alone.
        const int n0 = t.nkv0, n1 = TWO ? t.nkv : t.nkv0;  // one group: the loop is the first group's
        if (n0 == 1) umma_commit(&q_empty[0]);
        if (TWO && n1 == 1) umma_commit(&q_empty[1]);
        for (int j = 0; j < n1; ++j, ++it1) {
          const uint32_t iph0 = it0 & 1, iph1 = it1 & 1;
          const bool act0 = j < n0, more0 = j + 1 < n0, more1 = j + 1 < n1;
          const uint32_t vcur = kvs, vcur_ph = kvph;
          advance();
          uint32_t knext = 0, knext_ph = 0;
          if (more1) {
            knext = kvs;
            knext_ph = kvph;
            advance();
          }
          // PV0(j)
          if (!mbar_wait(&kv_full[vcur], vcur_ph, status, WAIT_SMEM_FULL)) { ok = false; break; }
          bool k_ready = more1 && mbar_test(&kv_full[knext], knext_ph);
          if (act0) {
            if (j == 0 && !mbar_wait(&o_free[0], tph ^ 1, status, WAIT_ATTN)) { ok = false; break; }
            if (!issue_pv(0, vcur, j > 0 ? 1u : 0u, iph0, mbar_test(&p_full[4 / ATT_PV_SLICES - 1], iph0), !more0)) { ok = false; break; }
            ++it0;
          }
          bool p1_ready = false;
          if (more1) {
            if (!k_ready && !mbar_wait(&kv_full[knext], knext_ph, status, WAIT_SMEM_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            if constexpr (TWO) p1_ready = mbar_test(&p_full[4 + 4 / ATT_PV_SLICES - 1], iph1);
            if (more0) {
              issue_qk(0, knext);
              if (j + 2 == n0) umma_commit(&q_empty[0]);
            }
          }
          // PV1(j)
          if constexpr (TWO) {
            if (j == 0 && !mbar_wait(&o_free[1], tph ^ 1, status, WAIT_ATTN)) { ok = false; break; }
            if (!issue_pv(1, vcur, j > 0 ? 1u : 0u, iph1, p1_ready, !more1)) { ok = false; break; }
          }
          umma_commit(&kv_empty[vcur]);
          if (more1) {
            if constexpr (TWO) issue_qk(1, knext);
            umma_commit(&kv_empty[knext]);
            if (TWO && j + 2 == n1) umma_commit(&q_empty[1]);
          }
        }
      }
    }
  } else if (warp < 4) {
    reg_dealloc<104>();  // warps 2 and 3 only take part in the warpgroup-wide register release
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    reg_alloc<192>();
    const int g = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row_in_group = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + g * S_COLS;
    const uint32_t t_o = tmem_base + lane_off + O_COL0 + g * D;
    const float scale = p.scale_log2;
    const int s_kv = p.s_kv, s_q = p.s_q, causal = p.causal;
    uint32_t it = 0, tcount = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok && (TWO || g == 0); unit += gridDim.x, ++tcount) {
      const AttnTile t = attn_tile<G>(p, unit);
      const int qrow = t.q0 + g * ATT_BM + row_in_group;  // position in the sequence
      float m = -INFINITY, l = 0.f;
      const int nkv_g = g == 0 ? t.nkv0 : t.nkv;
      for (int j = 0; j < nkv_g; ++j, ++it) {
        const uint32_t iph = it & 1;
        if (!mbar_wait(&s_full[g], iph, status, WAIT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        const int k0 = j * ATT_BN;
        // a block needs masking when it crosses the causal diagonal of this group or the KV tail
        const bool need_mask = (k0 + ATT_BN > s_kv) || (causal && (k0 + ATT_BN - 1 > t.q0 + g * ATT_BM));
        const int limit = causal ? min(s_kv - 1, qrow) : (s_kv - 1);  // last visible column
        // ---- the whole score row of this thread in registers: four loads in flight, one wait
        uint32_t sv[128];
        tmem_ld_row32<0>(t_s, sv);
        tmem_ld_row32<32>(t_s + 32, sv);
        tmem_ld_row32<64>(t_s + 64, sv);
        tmem_ld_row32<96>(t_s + 96, sv);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (k0 + i > limit) sv[i] = 0xff800000u;  // -inf: contributes exp2(-inf) = 0
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
          mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
        }
        const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;  // scale > 0
        float alpha = 1.f;
        if (j == 0) {
          m = m_blk;
        } else if (m_blk - m > ATT_RESCALE_THRESHOLD) {
          alpha = fast_exp2(m - m_blk);
          m = m_blk;
        }
        // ---- correction: rescale O_g when any row of this warp moved its reference max
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // PV_g(j-1) is complete: it precedes S_g(j) in the MMA stream, and S_g(j) has arrived
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_o + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32b_x32(t_o + c, v);
          }
          tmem_st_wait();
        }
        // ---- P = exp2(S * scale - m), row sum, packed 16-bit into the first half of S's columns
        const uint64_t scale2 = pack2(scale, scale);
        const uint64_t negm2 = pack2(-m, -m);
        uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 128; c += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x = fma2(pack2(__uint_as_float(sv[c + i]), __uint_as_float(sv[c + i + 1])), scale2, negm2);
            float x0, x1;
            unpack2(x, x0, x1);
            const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
            sum2 = add2(sum2, pack2(e0, e1));
            pk[i >> 1] = F16 ? pack_f16x2(e0, e1) : pack_bf16x2(e0, e1);
          }
          if (c > 0) {
            // the previous chunk's store has had this chunk's arithmetic to land: publish it
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&p_full[g * 4 + (c >> 5) - 1]);
          }
          tmem_st_32x32b_x16(t_s + (c >> 1), pk);
        }
        float sum_lo, sum_hi;
        unpack2(sum2, sum_lo, sum_hi);
        const float sum = sum_lo + sum_hi;
        l += sum;
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&p_full[g * 4 + 3]);
      }
      if (!ok) break;
      // ---- epilogue: wait for the last PV_g, normalise, store O and the base-2 LSE
      if (!mbar_wait(&pv_done[g], tcount & 1, status, WAIT_ATTN)) break;
      tc_fence_after_sync();
      const float inv_l = 1.f / l;
      const bool valid = qrow < s_q;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + ((size_t)t.bh * s_q + qrow) * D;
      // two tensor-memory loads in flight; O_g is handed back as soon as the last load has landed (before that
      // chunk is converted and stored); 32-byte stores when the row allows (each instruction writes whole sectors)
      const bool wide_st = (reinterpret_cast<uintptr_t>(orow) & 31) == 0;
      auto store32 = [&](const uint32_t (&v)[32], int c) {
        if (!valid) return;
        uint32_t w[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float lo = __uint_as_float(v[2 * u]) * inv_l;
          const float hi = __uint_as_float(v[2 * u + 1]) * inv_l;
          w[u] = F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
        }
        if (wide_st) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + c + 16 * i), "r"(w[8 * i]),
                         "r"(w[8 * i + 1]), "r"(w[8 * i + 2]), "r"(w[8 * i + 3]), "r"(w[8 * i + 4]), "r"(w[8 * i + 5]),
                         "r"(w[8 * i + 6]), "r"(w[8 * i + 7])
                         : "memory");
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(orow + c)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      };
      {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_o, v0);
#pragma unroll 1
        for (int c = 0; c < D; c += 64) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(t_o + c + 32, v1);
          store32(v0, c);
          tmem_ld_wait();
          if (c + 64 < D) {
            tmem_ld_32x32b_x32(t_o + c + 64, v0);
          } else {
            tc_fence_before_sync();
            mbar_arrive(&o_free[g]);
          }
          store32(v1, c + 32);
        }
      }
      if (valid && p.lse) p.lse[(size_t)t.bh * s_q + qrow] = m + log2f(l);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, int G>
static int launch_attn(const AttnParams& p, int grid, cudaStream_t stream) {
  using L = AttnSmem<D, G>;
  static_assert(L::TOTAL <= 232448, "shared memory budget");
  auto kfn = p.out_f16 ? attention_fwd_kernel<D, true, G> : attention_fwd_kernel<D, false, G>;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  kfn<<<grid, ATT_THREADS, L::TOTAL, stream>>>(p);
  return cuda_err(cudaGetLastError());
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_attention_fwd(const tb200_attention_args* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return TB200_ERR_BAD_ARG;
  if (a->batch < 0 || a->heads < 0 || a->seq_q < 0 || a->seq_kv < 0) return TB200_ERR_BAD_ARG;
  if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return TB200_ERR_UNSUPPORTED;
  if (a->dtype != TB200_BF16 && a->dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a->causal && a->seq_q != a->seq_kv) return TB200_ERR_UNSUPPORTED;
  if (!(a->sm_scale > 0.f)) return TB200_ERR_BAD_ARG;
  const long long bh = (long long)a->batch * a->heads;
  if (bh == 0 || a->seq_q == 0) return TB200_OK;
  if (a->seq_kv == 0) return TB200_ERR_BAD_ARG;
  if (bh > INT32_MAX || a->seq_q > (1 << 30) || a->seq_kv > (1 << 30)) return TB200_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->q) & 15) || (reinterpret_cast<uintptr_t>(a->k) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v) & 15) || (reinterpret_cast<uintptr_t>(a->o) & 15))
    return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  AttnParams p;
  memset(&p, 0, sizeof(p));
  const int D = a->head_dim;
  const CUtensorMapDataType dt =
      a->dtype == TB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint32_t box[3] = {64, 128, 1};
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->seq_q, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->seq_q * D * 2};
    int rc = encode_tmap(&p.tmq, dt, 3, a->q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)a->seq_kv, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)a->seq_kv * D * 2};
    int rc = encode_tmap(&p.tmk, dt, 3, a->k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap(&p.tmv, dt, 3, a->v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.o = a->o;
  p.lse = a->lse;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.bh = (int)bh;
  p.s_q = (int)a->seq_q;
  p.s_kv = (int)a->seq_kv;
  const int tile_rows = (D == 256 ? 1 : 2) * ATT_BM;
  p.q_tiles = (int)((a->seq_q + tile_rows - 1) / tile_rows);
  p.units = p.q_tiles * p.bh;
  p.causal = a->causal ? 1 : 0;
  p.out_f16 = a->dtype == TB200_F16 ? 1 : 0;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f;
  const int grid = p.units < sms ? p.units : sms;
  return D == 256 ? launch_attn<256, 1>(p, grid, stream)
         : D == 128 ? launch_attn<128, 2>(p, grid, stream) : launch_attn<64, 2>(p, grid, stream);
}
