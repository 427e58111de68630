// Flash-attention backward for sm_100a: dQ, dK, dV from Q, K, V, O, dO and the base-2
// log-sum-exp the forward kernel wrote.
//
// With s = Q K^T * sm_scale (masked), P = exp2(s * log2(e) - LSE2), Delta_i = sum_d O_id dO_id:
//   dV = P^T dO        dP = dO V^T        dS = P o (dP - Delta)
//   dK = sm_scale * dS^T Q                dQ = sm_scale * dS K
//
// One CTA owns one block of 128 KV rows of one (batch, head) and walks the query tiles (128 rows)
// that see it. Everything is computed transposed (KV rows on the 128 TMEM lanes) so that P^T and
// dS^T are the TMEM A operands of the dV and dK products. Five products per query tile j, each
// eight tcgen05.mma of N = 128 (measured on this part: an MMA costs about 45 cycles whatever its
// N below 128, 64-68 at N = 128, and the issuing thread pays ~70 cycles per barrier wait and ~30
// per commit, so few large instructions and few barriers per tile matter more than the overlap a
// second score buffer would buy):
//   S^T(j)  = K Q(j)^T        SS, 128 x 128 x D     -> TMEM S
//   dP^T(j) = V dO(j)^T       SS, 128 x 128 x D     -> TMEM dP
//   dV     += P^T(j) dO(j)    TS (P^T 16-bit, written over S), dO the MN-major B operand
//   dK     += dS^T(j) Q(j)    SS (dS^T from shared memory, K-major), Q the MN-major B operand
//   dQ^T(j) = K^T dS^T(j)     SS, both operands MN-major (K tile; the same dS^T tile),
//                             128 (d) x 128 (q) x 128 (kv), written over dP
// The per-query statistics enter through the MMAs: S^T and dP^T get a ninth K step whose B operand
// row q holds -LSE2[q] / scale (three 16-bit parts) and -Delta[q] (three parts) and whose A operand
// is a 0/1 selector, so the accumulators arrive as K Q^T - LSE2 / scale and dP^T - Delta and the
// compute groups need no per-column operand. (Reading the statistics inside their loops, from shared
// memory or by shuffle, cost 1000-1500 cycles per tile: such accesses crawl while SS MMAs stream
// their operands through the shared-memory pipe.)
// Tensor memory (512 columns): S (128) | dP (128) | dV (128) | dK (128).
// Roles (512 threads):
//   warp 0      TMA: K, V once; Q(j) through a three-deep ring of 128-row tiles, dO(j) through a single
//               buffer (dV(j) frees it early in the iteration; dP^T(j+1) needs it at the end).
//   warp 2      writes the statistics tile of each query tile (128 rows x 16 bytes).
//   warp 1      one thread issues every MMA, in the order
//                 dV(j) | S^T(j+1) | dQ^T(j), dK(j) | dP^T(j+1)
//               so that the exponentials of tile j+1 run under dQ^T, dK and dP^T, and dQ^T(j) is
//               read out of tensor memory while dK(j) executes.
//   warps 4-7   dQ reduction: read dQ^T(j) from TMEM (thread = head-dim column) and add it to the
//               fp32 dQ accumulator in global memory with coalesced red.add (a warp covers 128
//               contiguous bytes of one query row). Different KV blocks add to the same rows, so the
//               summation order - and the last bits of dQ - vary from run to run, as they do with
//               the reference's TMA reduce-add.
//   warps 8-11 / 12-15   compute groups 0 / 1 own query columns 0-63 / 64-127 of every tile; thread t
//               owns KV row t: P^T = exp2(scale * S') -> 16-bit -> TMEM (over the first 32 columns
//               of the group's half of S); dS^T = P^T o dP' -> 16-bit ->
//               shared memory, rows = kv with the 64 query columns of the group as one swizzled
//               128-byte row: read as the MN-major B operand by dQ^T and as the K-major A operand by
//               dK. dS^T is formed from the 16-bit P^T that dV also uses (32 registers instead of 64, which is
//               what lets the reduction group hold a whole dQ^T tile). The loops over a row are
//               branch-free (mask applied beforehand, dtype a template parameter): with a branch
//               per element pair they ran 1.6x slower, bound by MUFU latency instead of throughput.
//               At the end group 0 stores dV, group 1 stores sm_scale * dK.
// Registers per thread after setmaxnreg: 96 (load / MMA), 144 (dQ reduction, 128 of
// them one dQ^T row), 136 (compute groups).
// One thread's tcgen05.mma stream executes in order: S^T(j+1) may overwrite P^T(j) right after
// dV(j) was issued.
// Non-causal CTAs start their walk at a query tile that depends on the KV block, so that the CTAs
// of one head do not all add to the same dQ rows at the same time.
//
// Counterpart in the reference: _attn_bwd_preprocess, _attn_bwd_ws, _attn_bwd_dq_postprocess and
// _attention.backward, third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py
// :1252-1289, :2272-3283, :3362-3488.
#include <string.h>

#include "attention_common.cuh"
#include "common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int BWD_THREADS = 512;
static constexpr int BWD_BN = 128;  // kv rows per CTA
static constexpr int BWD_BM = 128;  // query rows per inner tile
static constexpr int BWD_D = 128;   // head dim
static constexpr int BWD_Q_STAGES = 3;   // Q(j) is read by S^T(j) early and by dK(j) late: a deep ring
// dO has a single buffer (freed by dV(j), refilled under S^T, dQ^T, dK)

struct AttnBwdParams {
  CUtensorMap tmq, tmdo;  // 3-D (D, S_q, B*H), box (64, 128, 1), 128-byte swizzle
  CUtensorMap tmk, tmv;   // 3-D (D, S_kv, B*H), box (64, 128, 1)
  const float* lse;       // [B*H, S_q] base-2
  const float* delta;     // [B*H, S_q]
  float* dq_acc;          // [B*H, S_q, D] fp32, zeroed before the launch
  void* dk;
  void* dv;
  int* status;
  int bh, s_q, s_kv;
  int kv_blocks;  // ceil(s_kv / 128)
  int q_tiles;    // ceil(s_q / 128)
  int causal;
  int f16;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

struct BwdSmem {
  static constexpr int KV_TILE = BWD_BN * BWD_D * 2;  // 32 KB
  static constexpr int Q_TILE = BWD_BM * BWD_D * 2;   // 32 KB
  static constexpr int DS_TILE = BWD_BN * BWD_BM * 2; // 32 KB: two 64-column groups of 16 KB
  static constexpr int K_OFFSET = 0;
  static constexpr int V_OFFSET = KV_TILE;
  static constexpr int Q_OFFSET = 2 * KV_TILE;
  static constexpr int DO_OFFSET = Q_OFFSET + BWD_Q_STAGES * Q_TILE;
  static constexpr int DS_OFFSET = DO_OFFSET + Q_TILE;
  // Row statistics ride on the MMAs as a ninth K step (see the header comment):
  static constexpr int AUG_B_OFFSET = DS_OFFSET + DS_TILE;      // [128 q] x 8 values, 16 bytes per row
  static constexpr int AUG_A_OFFSET = AUG_B_OFFSET + BWD_BM * 16;  // two selectors of 256 bytes
  static constexpr int BAR_OFFSET = AUG_A_OFFSET + 512;
  static constexpr int NUM_BARS = 2 + 2 * BWD_Q_STAGES + 2 + 2 + 6 + 1;
  // The tiles use all but a few hundred bytes of the 227 KB a CTA can have, so there is no room for
  // an alignment pad: the kernel checks that the dynamic window starts on a 1024-byte boundary.
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
};
static_assert(BwdSmem::TOTAL <= 232448, "shared memory budget");

struct BwdUnit {
  int bh, kv0, m_lo, m_cnt, rot;
};

__device__ __forceinline__ BwdUnit bwd_unit(const AttnBwdParams& p, int unit) {
  BwdUnit u;
  const int n = unit % p.kv_blocks;
  u.bh = unit / p.kv_blocks;
  u.kv0 = n * BWD_BN;
  if (p.causal) {
    u.m_lo = u.kv0 / BWD_BM;  // first query tile that reaches this KV block (BWD_BM == BWD_BN)
    u.m_cnt = max(p.q_tiles - u.m_lo, 0);
    u.rot = 0;
  } else {
    u.m_lo = 0;
    u.m_cnt = p.q_tiles;
    u.rot = n % p.q_tiles;
  }
  return u;
}
// query tile visited at step i of the walk
__device__ __forceinline__ int bwd_tile(const AttnBwdParams& p, const BwdUnit& u, int i) {
  int m = u.m_lo + i + u.rot;
  if (m >= p.q_tiles) m -= p.q_tiles;
  return m;
}

__device__ __forceinline__ void tmem_ld_row64(uint32_t taddr, uint32_t (&v)[64]) {
  tmem_ld_row32<0>(taddr, v);
  tmem_ld_row32<32>(taddr + 32, v);
}

template <bool F16>
__global__ void __launch_bounds__(BWD_THREADS, 1) attention_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using L = BwdSmem;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DP_COL0 = 128, DV_COL0 = 256, DK_COL0 = 384;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* k_full = bars;                       // [1]
  uint64_t* v_full = bars + 1;                   // [1]
  uint64_t* q_full = bars + 2;                   // [Q_STAGES]
  uint64_t* q_empty = q_full + BWD_Q_STAGES;     // [Q_STAGES]
  uint64_t* do_full = q_empty + BWD_Q_STAGES;    // [1]
  uint64_t* do_empty = do_full + 1;              // [1]
  uint64_t* aug_full = do_empty + 1;             // statistics warp -> MMA (32 arrivals)
  uint64_t* aug_empty = aug_full + 1;            // MMA -> statistics warp: dP^T(j) has read the tile
  uint64_t* s_full = aug_empty + 1;              // MMA -> compute: S^T ready
  uint64_t* p_full = s_full + 1;                 // compute -> MMA: P^T in TMEM (256 arrivals)
  uint64_t* dp_full = p_full + 1;                // MMA -> compute: dP^T ready
  uint64_t* ds_full = dp_full + 1;               // compute -> MMA: dS^T in TMEM and smem (256)
  uint64_t* dq_full = ds_full + 1;               // MMA -> reduce: dQ^T ready
  uint64_t* dq_empty = dq_full + 1;              // reduce -> MMA: dQ^T read out (128)
  uint64_t* dkv_done = dq_empty + 1;             // MMA -> compute: dV, dK complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dkv_done + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  if (smem_a & 1023u) {  // the swizzled tiles need a 1024-byte aligned window (uniform over the CTA)
    if (threadIdx.x == 0) atomicCAS(status, 0, (BAD_SMEM_ALIGNMENT << 16) | (int)(blockIdx.x & 0xffff));
    return;
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmq);
    tma_prefetch_desc(&p.tmdo);
    tma_prefetch_desc(&p.tmk);
    tma_prefetch_desc(&p.tmv);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    for (int i = 0; i < BWD_Q_STAGES; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(aug_full, 32);
    mbar_init(aug_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 256);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 128);
    mbar_init(dkv_done, 1);
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
  const BwdUnit u = bwd_unit(p, blockIdx.x);
  const int n_tiles = u.m_cnt;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    reg_dealloc<96>();
    if (lane == 0) {
      const uint64_t pol_kv = policy_evict_first();  // read once by this CTA
      const uint64_t pol_q = policy_evict_last();    // re-read by every KV block of the head
      auto load_tile = [&](const CUtensorMap* tm, uint32_t off, uint64_t* bar, int row, uint64_t pol) {
        mbar_expect_tx(bar, L::KV_TILE);
        tma_load_3d(smem + off, tm, bar, 0, row, u.bh, pol);
        tma_load_3d(smem + off + L::KV_TILE / 2, tm, bar, 64, row, u.bh, pol);
      };
      load_tile(&p.tmk, L::K_OFFSET, k_full, u.kv0, pol_kv);
      uint32_t qs = 0, qph = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int q0 = bwd_tile(p, u, j) * BWD_BM;
        if (!mbar_wait(&q_empty[qs], qph ^ 1, status, WAIT_SMEM_EMPTY)) break;
        load_tile(&p.tmq, L::Q_OFFSET + qs * L::Q_TILE, &q_full[qs], q0, pol_q);
        if (j == 0) load_tile(&p.tmv, L::V_OFFSET, v_full, u.kv0, pol_kv);
        if (!mbar_wait(do_empty, (j & 1) ^ 1, status, WAIT_SMEM_EMPTY)) break;
        load_tile(&p.tmdo, L::DO_OFFSET, do_full, q0, pol_q);
        if (++qs == BWD_Q_STAGES) { qs = 0; qph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    reg_dealloc<96>();
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t fmt_fix = F16 ? ((1u << 7) | (1u << 10)) : 0u;  // fp16: operand format 0
      const uint32_t id_st = make_idesc(1u, 1u, 0u, 0u, BWD_BN, BWD_BM) & ~fmt_fix;  // K-major x K-major
      const uint32_t id_acc = make_idesc(1u, 1u, 0u, 1u, BWD_BN, BWD_D) & ~fmt_fix;  // TMEM A, MN-major B
      const uint32_t id_dq = make_idesc(1u, 1u, 1u, 1u, BWD_D, BWD_BM) & ~fmt_fix;   // MN-major x MN-major
      constexpr uint32_t HALF = L::KV_TILE / 2;  // one 64-column box of a 128-row tile
      const uint64_t k_kmaj = make_smem_desc(smem_a + L::K_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t v_kmaj = make_smem_desc(smem_a + L::V_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t k_mnmaj = make_smem_desc(smem_a + L::K_OFFSET, HALF, 1024, SWIZZLE_128B);
      const uint64_t q_kmaj0 = make_smem_desc(smem_a + L::Q_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t q_mnmaj0 = make_smem_desc(smem_a + L::Q_OFFSET, HALF, 1024, SWIZZLE_128B);
      const uint64_t do_kmaj0 = make_smem_desc(smem_a + L::DO_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t do_mnmaj0 = make_smem_desc(smem_a + L::DO_OFFSET, HALF, 1024, SWIZZLE_128B);
      const uint64_t ds_mnmaj = make_smem_desc(smem_a + L::DS_OFFSET, HALF, 1024, SWIZZLE_128B);
      const uint64_t ds_kmaj = make_smem_desc(smem_a + L::DS_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint32_t id_dk = make_idesc(1u, 1u, 0u, 1u, BWD_BN, BWD_D) & ~fmt_fix;  // K-major A (smem), MN-major B
      // ninth K step (unswizzled K-major core matrices of 8 rows x 16 bytes): the B operand has one
      // 16-byte row per query (both K halves alias it: leading byte offset 0), the A operand is one
      // 8-row selector repeated down the 128 kv rows (stride byte offset 0)
      const uint64_t aug_b = make_smem_desc(smem_a + L::AUG_B_OFFSET, 0, 128, SWIZZLE_NONE);
      const uint64_t aug_a_s = make_smem_desc(smem_a + L::AUG_A_OFFSET, 128, 0, SWIZZLE_NONE);
      const uint64_t aug_a_dp = make_smem_desc(smem_a + L::AUG_A_OFFSET + 256, 128, 0, SWIZZLE_NONE);
      bool ok = true;

      // S^T or dP^T: [128 kv] x [128 q] over D, both operands K-major, plus the statistics step
      auto issue_kq = [&](uint64_t a_desc, uint64_t b_desc, uint32_t d_col, uint64_t a_aug) {
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t o = (uint64_t)(((k >> 2) * HALF + (k & 3) * 32) >> 4);
          umma_f16_ss(tmem_base + d_col, a_desc + o, b_desc + o, id_st, k > 0 ? 1u : 0u);
        }
        umma_f16_ss(tmem_base + d_col, a_aug, aug_b, id_st, 1u);
      };
      // dV += P^T dO: A = 16-bit [128 kv] x [128 q] in TMEM (32 columns at 0 and 32 at 64),
      // B = dO as [128 q] x [128 d]
      auto issue_dv = [&](uint64_t b_desc, uint32_t accum) {
#pragma unroll
        for (int k = 0; k < BWD_BM / 16; ++k)
          umma_f16_ts(tmem_base + DV_COL0, tmem_base + (k >> 2) * 64 + (k & 3) * 8,
                      b_desc + (uint64_t)((k * 2048) >> 4), id_acc, k > 0 ? 1u : accum);
      };
      // dK += dS^T Q: A = dS^T from shared memory (K-major: rows kv, q contiguous), B = Q as [128 q] x [128 d]
      auto issue_dk = [&](uint64_t b_desc, uint32_t accum) {
#pragma unroll
        for (int k = 0; k < BWD_BM / 16; ++k)
          umma_f16_ss(tmem_base + DK_COL0, ds_kmaj + (uint64_t)(((k >> 2) * HALF + (k & 3) * 32) >> 4),
                      b_desc + (uint64_t)((k * 2048) >> 4), id_dk, k > 0 ? 1u : accum);
      };
      // dQ^T = K^T dS^T: [128 d] x [128 q] over the 128 kv rows
      auto issue_dq = [&]() {
#pragma unroll
        for (int k = 0; k < BWD_BN / 16; ++k) {
          const uint64_t o = (uint64_t)((k * 2048) >> 4);
          umma_f16_ss(tmem_base + DP_COL0, k_mnmaj + o, ds_mnmaj + o, id_dq, k > 0 ? 1u : 0u);
        }
      };

      // prologue: S^T(0), dP^T(0)
      ok = mbar_wait(k_full, 0, status, WAIT_SMEM_FULL) && mbar_wait(&q_full[0], 0, status, WAIT_SMEM_FULL) &&
           mbar_wait(aug_full, 0, status, WAIT_SMEM_FULL);
      if (ok) {
        tc_fence_after_sync();
        issue_kq(k_kmaj, q_kmaj0, 0, aug_a_s);
        umma_commit(s_full);
        ok = mbar_wait(v_full, 0, status, WAIT_SMEM_FULL) && mbar_wait(do_full, 0, status, WAIT_SMEM_FULL);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_kq(v_kmaj, do_kmaj0, DP_COL0, aug_a_dp);
        umma_commit(dp_full);
        umma_commit(aug_empty);
      }
      bool p_ready = false;
      uint32_t qs = 0, qph = 0;  // ring position of Q(j)
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = j & 1;
        const uint64_t st_off = (uint64_t)((qs * L::Q_TILE) >> 4);
        uint32_t qs1 = qs + 1, qph1 = qph;
        if (qs1 == BWD_Q_STAGES) { qs1 = 0; qph1 ^= 1; }
        const uint64_t st1_off = (uint64_t)((qs1 * L::Q_TILE) >> 4);
        const bool more = j + 1 < n_tiles;
        // Each barrier is probed (test_wait) ahead of the MMA batch that precedes its use: a blocking
        // wait costs this thread ~70 cycles even when the phase is already complete.
        // dV += P^T(j) dO(j)
        if (!p_ready && !mbar_wait(p_full, ph, status, WAIT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        bool q_ready = more && mbar_test(&q_full[qs1], qph1) && mbar_test(aug_full, ph ^ 1);
        issue_dv(do_mnmaj0, j > 0 ? 1u : 0u);
        umma_commit(do_empty);
        // S^T(j+1) over P^T(j)
        bool ds_ready = false;
        if (more) {
          if (!q_ready && !(mbar_wait(&q_full[qs1], qph1, status, WAIT_SMEM_FULL) &&
                            mbar_wait(aug_full, ph ^ 1, status, WAIT_SMEM_FULL))) { ok = false; break; }
          tc_fence_after_sync();
          ds_ready = mbar_test(ds_full, ph);
          issue_kq(k_kmaj, q_kmaj0 + st1_off, 0, aug_a_s);
          umma_commit(s_full);
        }
        // dQ^T(j) = K^T dS^T(j) over dP^T(j); then dK += dS^T(j) Q(j) while the reduction group
        // reads dQ^T(j) out
        if (!ds_ready && !mbar_wait(ds_full, ph, status, WAIT_ATTN)) { ok = false; break; }
        tc_fence_after_sync();
        bool do_ready = more && mbar_test(do_full, ph ^ 1);
        issue_dq();
        umma_commit(dq_full);
        issue_dk(q_mnmaj0 + st_off, j > 0 ? 1u : 0u);
        umma_commit(&q_empty[qs]);
        // dP^T(j+1), once dQ^T(j) has left those columns
        p_ready = false;
        if (more) {
          if (!do_ready && !mbar_wait(do_full, ph ^ 1, status, WAIT_SMEM_FULL)) { ok = false; break; }
          if (!mbar_wait(dq_empty, ph, status, WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after_sync();
          p_ready = mbar_test(p_full, ph ^ 1);
          issue_kq(v_kmaj, do_kmaj0, DP_COL0, aug_a_dp);
          umma_commit(dp_full);
          umma_commit(aug_empty);
        }
        qs = qs1;
        qph = qph1;
      }
      if (ok) umma_commit(dkv_done);
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ row statistics
    reg_dealloc<96>();
    // selectors: ones in K columns 0-2 (S^T step) / 3-5 (dP^T step) of the first K half, zero elsewhere
    {
      const uint16_t one = F16 ? 0x3C00 : 0x3F80;
      uint16_t* a = reinterpret_cast<uint16_t*>(smem + L::AUG_A_OFFSET);
      for (int i = lane; i < 256; i += 32) {  // 2 selectors x 2 core matrices x 8 rows x 8 values
        const int sel = i >> 7, half = (i >> 6) & 1, col = i & 7;
        a[i] = (half == 0 && col >= 3 * sel && col < 3 * sel + 3) ? one : (uint16_t)0;
      }
    }
    const float inv_scale = 1.f / p.scale_log2;
    for (int j = 0; j < n_tiles; ++j) {
      const int q0 = bwd_tile(p, u, j) * BWD_BM;
      // a query row past the end gets zeros: S' = 0, P = 1, and its dO row and Delta are zero, so it
      // contributes nothing. The loads are issued before the wait for the buffer.
      float vals[BWD_BM / 32][2];
#pragma unroll
      for (int h = 0; h < BWD_BM / 32; ++h) {
        const int q = q0 + lane + 32 * h;
        vals[h][0] = 0.f;
        vals[h][1] = 0.f;
        if (q < p.s_q) {
          const size_t idx = (size_t)u.bh * p.s_q + q;
          vals[h][0] = -__ldg(p.lse + idx) * inv_scale;
          vals[h][1] = -__ldg(p.delta + idx);
        }
      }
      // the tile of step j-1 was last read by dP^T(j-1)
      if (!mbar_wait(aug_empty, (j & 1) ^ 1, status, WAIT_SMEM_EMPTY)) break;
#pragma unroll
      for (int h = 0; h < BWD_BM / 32; ++h) {
        // each value as three 16-bit parts (hi + mid + lo, ~24 bits together); the MMA multiplies
        // them by 1 and adds them in fp32
        uint16_t w[8];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          float rem = vals[h][t];
#pragma unroll
          for (int part = 0; part < 3; ++part) {
            float back;
            if (F16) {
              const __half hv = __float2half_rn(rem);
              w[3 * t + part] = __half_as_ushort(hv);
              back = __half2float(hv);
            } else {
              const __nv_bfloat16 bv = __float2bfloat16_rn(rem);
              w[3 * t + part] = __bfloat16_as_ushort(bv);
              back = __bfloat162float(bv);
            }
            rem -= back;
          }
        }
        w[6] = 0;
        w[7] = 0;
        *reinterpret_cast<uint4*>(smem + L::AUG_B_OFFSET + (lane + 32 * h) * 16) =
            make_uint4(w[0] | ((uint32_t)w[1] << 16), w[2] | ((uint32_t)w[3] << 16), w[4] | ((uint32_t)w[5] << 16),
                       w[6] | ((uint32_t)w[7] << 16));
      }
      fence_proxy_async_smem();
      mbar_arrive(aug_full);
    }
  } else if (warp == 3) {
    reg_dealloc<96>();  // takes part in the warpgroup-wide register release only
  } else if (warp < 8) {
    // ------------------------------------------------------------------ dQ reduction
    reg_alloc<144>();
    const int qd = warp & 3;
    const int d = qd * 32 + lane;
    const uint32_t t_dq = tmem_base + ((uint32_t)(qd * 32) << 16) + DP_COL0;
    for (int j = 0; j < n_tiles; ++j) {
      const int q0 = bwd_tile(p, u, j) * BWD_BM;
      if (!mbar_wait(dq_full, j & 1, status, WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      float* dst = p.dq_acc + ((size_t)u.bh * p.s_q + q0) * BWD_D + d;
      const int valid = min(BWD_BM, p.s_q - q0);
      uint32_t v[128];
      tmem_ld_row32<0>(t_dq, v);
      tmem_ld_row32<32>(t_dq + 32, v);
      tmem_ld_row32<64>(t_dq + 64, v);
      tmem_ld_row32<96>(t_dq + 96, v);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(dq_empty);  // the whole tile is in registers: the columns are free for dP^T(j+1)
#pragma unroll
      for (int c = 0; c < BWD_BM; ++c)
        if (c < valid) atomicAdd(dst + (size_t)c * BWD_D, __uint_as_float(v[c]));
    }
  } else {
    // ------------------------------------------------------------------ compute groups
    reg_alloc<136>();
    const int g = (warp - 8) >> 2;  // query columns 64 g .. 64 g + 63 of every tile
    const int qd = warp & 3;
    const int r = qd * 32 + lane;  // kv row of this thread within the block
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const uint32_t t_s = tmem_base + lane_off + g * 64;
    const uint32_t t_dp = tmem_base + lane_off + DP_COL0 + g * 64;
    uint8_t* ds_row = smem + L::DS_OFFSET + g * (L::DS_TILE / 2) + r * 128;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t ph = j & 1;
      const int q0 = bwd_tile(p, u, j) * BWD_BM + g * 64;
      if (!mbar_wait(s_full, ph, status, WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t pp[32];  // P^T of this tile as stored (16-bit pairs); dS^T is formed from these values
      uint32_t pk[32];
      {
        uint32_t sv[64];
        tmem_ld_row64(t_s, sv);
        tmem_ld_wait();
        // under the causal mask a query column is visible when q0 + c >= kv0 + r; a masked score
        // becomes -inf before the (branch-free) exponential loop: exp2(-inf * scale - LSE2) = 0
        if (p.causal && (q0 < u.kv0 + BWD_BN - 1)) {
          const int lim = u.kv0 + r - q0;
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c < lim) sv[c] = 0xff800000u;
        }
        // S' already holds K Q^T - LSE2 / scale (ninth K step), so P^T = exp2(scale * S')
        const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float x0, x1;
          unpack2(mul2(pack2(__uint_as_float(sv[2 * c]), __uint_as_float(sv[2 * c + 1])), scale2), x0, x1);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          pp[c] = F16 ? pack_f16x2(e0, e1) : pack_bf16x2(e0, e1);
        }
      }
      tmem_st_32x32b_x32(t_s, pp);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      // dS^T = P^T o (dP^T - Delta), 16-bit, into shared memory: rows = kv, 64 query columns of this
      // group as one 128-byte swizzled row (the MN-major B operand of dQ^T and the K-major A operand of dK)
      if (!mbar_wait(dp_full, ph, status, WAIT_ATTN)) { ok = false; break; }
      tc_fence_after_sync();
      {
        uint32_t dv[64];
        tmem_ld_row64(t_dp, dv);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {  // one 16-byte chunk of the dS^T row: 8 query columns
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const int c = 4 * ch + h;
            float p0, p1;  // dP' already holds dP^T - Delta (ninth K step)
            unpack2(unpack16x2<F16>(pp[c]), p0, p1);
            const float a0 = p0 * __uint_as_float(dv[2 * c]);
            const float a1 = p1 * __uint_as_float(dv[2 * c + 1]);
            pk[c] = F16 ? pack_f16x2(a0, a1) : pack_bf16x2(a0, a1);
          }
          *reinterpret_cast<uint4*>(ds_row + ((ch ^ (r & 7)) << 4)) =
              make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();  // orders this thread's reads of dP^T before the dQ^T MMA that overwrites them
      mbar_arrive(ds_full);
    }
    // ---- epilogue: group 0 stores dV, group 1 stores sm_scale * dK
    const int kv = u.kv0 + r;
    uint16_t* orow = reinterpret_cast<uint16_t*>(g == 0 ? p.dv : p.dk) + ((size_t)u.bh * p.s_kv + kv) * BWD_D;
    const float oscale = g == 0 ? 1.f : p.sm_scale;
    const uint32_t t_acc = tmem_base + lane_off + (g == 0 ? DV_COL0 : DK_COL0);
    if (n_tiles > 0) ok = ok && mbar_wait(dkv_done, 0, status, WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < BWD_D; c += 32) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32b_x32(t_acc + c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (kv < p.s_kv) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float lo = __uint_as_float(v[i * 8 + 2 * t]) * oscale;
              const float hi = __uint_as_float(v[i * 8 + 2 * t + 1]) * oscale;
              w[t] = F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
            }
            reinterpret_cast<uint4*>(orow + c)[i] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Delta[row] = sum_d O[row, d] * dO[row, d]; one warp per row, D = 128 (4 elements per lane).
template <typename T>
__global__ void attention_bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                           float* __restrict__ delta, long long rows) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 a = reinterpret_cast<const uint2*>(o + row * BWD_D)[lane];
  const uint2 b = reinterpret_cast<const uint2*>(d_o + row * BWD_D)[lane];
  const T* av = reinterpret_cast<const T*>(&a);
  const T* bv = reinterpret_cast<const T*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) s += static_cast<float>(av[i]) * static_cast<float>(bv[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[row] = s;
}

// dQ = sm_scale * accumulator, converted to the 16-bit output type; 8 elements per thread.
template <typename T>
__global__ void attention_bwd_dq_kernel(const float* __restrict__ acc, T* __restrict__ dq, long long n8,
                                        float sm_scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 x = reinterpret_cast<const float4*>(acc)[2 * i];
  const float4 y = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  const float v[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
  uint4 out;
  T* ov = reinterpret_cast<T*>(&out);
#pragma unroll
  for (int j = 0; j < 8; ++j) ov[j] = static_cast<T>(v[j] * sm_scale);
  reinterpret_cast<uint4*>(dq)[i] = out;
}

static size_t bwd_delta_bytes(long long rows) { return (((size_t)rows * 4) + 255) & ~(size_t)255; }

}  // namespace tb200

using namespace tb200;

static int bwd_validate(const tb200_attention_bwd_args* a) {
  if (!a) return TB200_ERR_BAD_ARG;
  if (a->batch < 0 || a->heads < 0 || a->seq_q < 0 || a->seq_kv < 0) return TB200_ERR_BAD_ARG;
  if (a->head_dim != BWD_D) return TB200_ERR_UNSUPPORTED;
  if (a->dtype != TB200_BF16 && a->dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a->causal && a->seq_q != a->seq_kv) return TB200_ERR_UNSUPPORTED;
  const long long bh = (long long)a->batch * a->heads;
  if (bh > INT32_MAX || a->seq_q > (1 << 30) || a->seq_kv > (1 << 30)) return TB200_ERR_UNSUPPORTED;
  return TB200_OK;
}

extern "C" size_t tb200_attention_bwd_workspace_bytes(const tb200_attention_bwd_args* a) {
  if (bwd_validate(a) != TB200_OK) return 0;
  const long long rows = (long long)a->batch * a->heads * a->seq_q;
  return bwd_delta_bytes(rows) + (size_t)rows * BWD_D * 4;
}

extern "C" int tb200_attention_bwd(const tb200_attention_bwd_args* a, void* stream_) {
  int rc = bwd_validate(a);
  if (rc != TB200_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->d_o || !a->lse || !a->dq || !a->dk || !a->dv) return TB200_ERR_BAD_ARG;
  if (!(a->sm_scale > 0.f)) return TB200_ERR_BAD_ARG;
  const long long bh = (long long)a->batch * a->heads;
  if (bh == 0 || (a->seq_q == 0 && a->seq_kv == 0)) return TB200_OK;
  if (a->seq_q == 0 || a->seq_kv == 0) return TB200_ERR_BAD_ARG;
  const void* ptrs[] = {a->q, a->k, a->v, a->o, a->d_o, a->dq, a->dk, a->dv, a->workspace};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return TB200_ERR_BAD_ARG;
  const size_t need = tb200_attention_bwd_workspace_bytes(a);
  if (!a->workspace || a->workspace_bytes < need) return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long rows = bh * a->seq_q;
  const long long kv_blocks = (a->seq_kv + BWD_BN - 1) / BWD_BN;
  if (bh * kv_blocks > INT32_MAX) return TB200_ERR_UNSUPPORTED;

  float* delta = static_cast<float*>(a->workspace);
  float* dq_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + bwd_delta_bytes(rows));

  AttnBwdParams p;
  memset(&p, 0, sizeof(p));
  const bool f16 = a->dtype == TB200_F16;
  const CUtensorMapDataType dt = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  {
    const uint32_t box[3] = {64, BWD_BM, 1};
    const uint64_t dims[3] = {(uint64_t)BWD_D, (uint64_t)a->seq_q, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)BWD_D * 2, (uint64_t)a->seq_q * BWD_D * 2};
    rc = encode_tmap(&p.tmq, dt, 3, a->q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap(&p.tmdo, dt, 3, a->d_o, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    const uint32_t box[3] = {64, BWD_BN, 1};
    const uint64_t dims[3] = {(uint64_t)BWD_D, (uint64_t)a->seq_kv, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)BWD_D * 2, (uint64_t)a->seq_kv * BWD_D * 2};
    rc = encode_tmap(&p.tmk, dt, 3, a->k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap(&p.tmv, dt, 3, a->v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.lse = a->lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = a->dk;
  p.dv = a->dv;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.bh = (int)bh;
  p.s_q = (int)a->seq_q;
  p.s_kv = (int)a->seq_kv;
  p.kv_blocks = (int)kv_blocks;
  p.q_tiles = (int)((a->seq_q + BWD_BM - 1) / BWD_BM);
  p.causal = a->causal ? 1 : 0;
  p.f16 = f16 ? 1 : 0;
  p.sm_scale = a->sm_scale;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f;

  // 1. Delta = rowsum(O o dO);  2. zero the fp32 dQ accumulator
  {
    const int warps = 8;
    const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
    if (f16)
      attention_bwd_delta_kernel<__half><<<blocks, warps * 32, 0, stream>>>(
          static_cast<const __half*>(a->o), static_cast<const __half*>(a->d_o), delta, rows);
    else
      attention_bwd_delta_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(a->o), static_cast<const __nv_bfloat16*>(a->d_o), delta, rows);
    rc = cuda_err(cudaGetLastError());
    if (rc != TB200_OK) return rc;
    rc = cuda_err(cudaMemsetAsync(dq_acc, 0, (size_t)rows * BWD_D * 4, stream));
    if (rc != TB200_OK) return rc;
  }
  // 3. the main kernel: one CTA per (batch*head, KV block)
  {
    auto kfn = f16 ? attention_bwd_kernel<true> : attention_bwd_kernel<false>;
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL) != cudaSuccess)
      return TB200_ERR_CUDA;
    kfn<<<(unsigned)(bh * kv_blocks), BWD_THREADS, BwdSmem::TOTAL, stream>>>(p);
    rc = cuda_err(cudaGetLastError());
    if (rc != TB200_OK) return rc;
  }
  // 4. dQ = sm_scale * accumulator
  {
    const long long n8 = rows * BWD_D / 8;
    const unsigned blocks = (unsigned)((n8 + 255) / 256);
    if (f16)
      attention_bwd_dq_kernel<__half><<<blocks, 256, 0, stream>>>(dq_acc, static_cast<__half*>(a->dq), n8, a->sm_scale);
    else
      attention_bwd_dq_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(a->dq),
                                                                         n8, a->sm_scale);
    rc = cuda_err(cudaGetLastError());
  }
  return rc;
}
