// MXFP8 flash-attention forward for sm_100a: O = softmax(dq(Q) dq(K)^T * sm_scale [+ causal mask]) dq(V) with Q, K, V
// in e4m3 and one e8m0 scale per 32 values - Q and K scaled along the head dimension, V along the sequence (its
// transpose is what was quantised), P quantised by the kernel per 32 keys - and both products on the block-scaled
// tensor cores (tcgen05.mma.kind::mxf8f6f4.block_scale, K = 32 per instruction).
//
// One CTA handles 128 query rows of one (batch, head); KV is walked in blocks of 128. Roles (256 threads):
//   warp 0     TMA: Q tile + its scale atom once per tile; K(j), V(j) and their scale atoms through a 3-deep ring.
//   warp 1     one thread issues every MMA: S(j) = Q K(j)^T (SS, four K = 32 steps over the head dimension) into one
//              of two score buffers, so that S(j+1) is computed while the softmax works on S(j); then, when P(j) is
//              published, O += P(j) V(j) (SS: P from shared memory, V the MN-major B operand, four steps over the
//              128 keys). Scale atoms (512 bytes: [row % 32][row / 32][block]) go to tensor memory by tcgen05.cp.
//   warps 4-11 softmax: two threads per query row (64 score columns each). Online softmax in the exp2 domain with the lazy rescale of the
//              16-bit kernel (the accumulator is rescaled only when a row's maximum grew by more than 2^8);
//              p = exp2(s * scale - m) in fp32, its row sum in fp32; every 32 keys of a row share the e8m0 scale
//              2^ceil(log2(amax / 448)), p / scale is rounded to e4m3 and written to shared memory in the 128-byte
//              swizzled K-major layout the MMA descriptor expects, the four scale bytes of the row into an atom.
//              P and its atom are double-buffered, so the softmax of block j+1 runs while P(j) V(j) executes;
//              At the end: O / l as bf16 and the base-2 log-sum-exp.
// Tensor memory (512 columns allocated): S0 | S1 | O | scale columns (Q 4; P, K, V two sets of 4 each).
// One query group per CTA. A variant with two groups of 128 rows per CTA sharing every K / V tile (one score buffer
// handed back and forth, since tensor memory cannot hold two score buffers, two accumulators and the scale
// columns) measured the same or slower (992 against 1030 TFLOP/s at [4, 32, 8192, 128]): with the scores and P
// double-buffered the tensor pipe already runs under the softmax, and the softmax itself is bound by the
// special-function unit, which serves the exponentials and the e4m3 conversions of both groups alike. Two threads
// per query row (this version) gained 2-10 % over one; requesting the next block's scores from tensor memory
// while the current block is worked on lost 25 % (the second row buffer spills).
//
// Counterpart in the reference: _attn_fwd_mxf8_ws and its host entry `attention(q, k, v, q_scale, k_scale, v_scale,
// sm_scale, causal)`, third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent_mxfp8.py:532-1130, :3374
// (P quantisation third_party/tlx/language/tlx/mxfp8_utils.py:224-302).
#include <string.h>

#include "attention_common.cuh"
#include "common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int MXA_THREADS = 384;  // TMA warp, MMA warp, two idle, eight softmax warps (two threads per query row)
static constexpr int MXA_BM = 128;
static constexpr int MXA_BN = 128;
static constexpr int MXA_D = 128;
static constexpr int MXA_STAGES = 3;
static constexpr float MXA_RESCALE_THRESHOLD = 8.0f;

struct MxAttnParams {
  CUtensorMap tmq, tmk, tmv;  // 3-D (D bytes, S, B*H) uint8, box (128, 128, 1), 128-byte swizzle
  const uint8_t* sfq;         // atoms [B*H][S_q / 128][512]
  const uint8_t* sfk;         // atoms [B*H][S_kv / 128][512]
  const uint8_t* sfv;         // atoms [B*H][S_kv / 128][512]: rows = head-dim columns, blocks = 32-key groups
  void* o;                    // bf16 [B, H, S_q, D]
  float* lse;
  int* status;
  int bh, s_q, s_kv, q_tiles, units, causal, head_major;
  float scale_log2;
};

struct MxAttnSmem {
  static constexpr int TILE = 128 * 128;  // one 128-row tile of fp8
  static constexpr int Q_OFFSET = 0;
  static constexpr int KV_OFFSET = TILE;                              // ring: K tile, V tile per stage
  static constexpr int P_OFFSET = KV_OFFSET + MXA_STAGES * 2 * TILE;  // two P tiles
  static constexpr int SF_OFFSET = P_OFFSET + 2 * TILE;               // atoms: Q | P0 | P1 | (K, V) per stage
  static constexpr int XCHG_OFFSET = SF_OFFSET + (3 + 2 * MXA_STAGES) * 512;  // [parity][half][row] floats
  static constexpr int BAR_OFFSET = XCHG_OFFSET + 2 * 2 * 128 * 4;
  static constexpr int NUM_BARS = 2 + 2 * MXA_STAGES + 2 + 2 + 2 + 1;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;
};

__device__ __forceinline__ void mxa_tile(const MxAttnParams& p, int unit, int& bh, int& q0, int& nkv) {
  int qb;
  if (p.head_major) {  // all query tiles of a head side by side: its K / V stream is shared through L2
    bh = unit / p.q_tiles;
    qb = p.q_tiles - 1 - unit % p.q_tiles;
  } else {             // longest (causal) tiles first, heads side by side
    qb = p.q_tiles - 1 - unit / p.bh;
    bh = unit % p.bh;
  }
  q0 = qb * MXA_BM;
  nkv = (p.s_kv + MXA_BN - 1) / MXA_BN;
  if (p.causal) nkv = min(nkv, (q0 + MXA_BM + MXA_BN - 1) / MXA_BN);
}

__global__ void __launch_bounds__(MXA_THREADS, 1) attention_mxfp8_fwd_kernel(const __grid_constant__ MxAttnParams p) {
  using L = MxAttnSmem;
  constexpr uint32_t S_COL0 = 0, O_COL = 256;
  constexpr uint32_t SFQ_COL = 384, SFP_COL0 = 388, SFK_COL0 = 396, SFV_COL0 = 404;  // P, K, V: two sets of 4
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* q_full = bars;                         // loader -> MMA
  uint64_t* q_empty = bars + 1;                    // MMA -> loader (commit after the tile's last S)
  uint64_t* kv_full = bars + 2;                    // [STAGES]
  uint64_t* kv_empty = kv_full + MXA_STAGES;       // [STAGES] commit after PV(j)
  uint64_t* s_full = kv_empty + MXA_STAGES;        // [2] MMA -> softmax
  uint64_t* p_full = s_full + 2;                   // [2] softmax -> MMA (128 arrivals): P tile n (buffer n & 1) and its scales are in shared memory
  uint64_t* pv_done = p_full + 2;                  // [2] MMA -> softmax: the product with P tile n is complete (O updated, buffer n & 1 free)
  uint64_t* o_free = pv_done + 2;                  // softmax -> MMA (128 arrivals): O read out, the next tile may start
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmq);
    tma_prefetch_desc(&p.tmk);
    tma_prefetch_desc(&p.tmv);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < MXA_STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_full[i], 256);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(o_free, 256);
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
  const int kv_blocks_per_head = (p.s_kv + MXA_BN - 1) / MXA_BN;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      const uint64_t pol_q = policy_evict_first();
      const uint64_t pol_kv = policy_evict_last();
      uint32_t kvs = 0, kvph = 0, tcount = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
        int bh, q0, nkv;
        mxa_tile(p, unit, bh, q0, nkv);
        if (!mbar_wait(q_empty, (tcount & 1) ^ 1, status, WAIT_SMEM_EMPTY)) break;
        mbar_expect_tx(q_full, L::TILE + 512);
        tma_load_3d(smem + L::Q_OFFSET, &p.tmq, q_full, 0, q0, bh, pol_q);
        bulk_load(smem + L::SF_OFFSET, p.sfq + ((size_t)bh * p.q_tiles + q0 / MXA_BM) * 512, 512, q_full);
        for (int j = 0; j < nkv; ++j) {
          if (!mbar_wait(&kv_empty[kvs], kvph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&kv_full[kvs], 2 * L::TILE + 1024);
          uint8_t* kt = smem + L::KV_OFFSET + kvs * 2 * L::TILE;
          tma_load_3d(kt, &p.tmk, &kv_full[kvs], 0, j * MXA_BN, bh, pol_kv);
          tma_load_3d(kt + L::TILE, &p.tmv, &kv_full[kvs], 0, j * MXA_BN, bh, pol_kv);
          uint8_t* sf = smem + L::SF_OFFSET + (3 + 2 * kvs) * 512;
          const size_t atom = ((size_t)bh * kv_blocks_per_head + j) * 512;
          bulk_load(sf, p.sfk + atom, 512, &kv_full[kvs]);
          bulk_load(sf + 512, p.sfv + atom, 512, &kv_full[kvs]);
          if (++kvs == MXA_STAGES) {
            kvs = 0;
            kvph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t id_qk[4], id_pv[4];
#pragma unroll
      for (uint32_t k = 0; k < 4; ++k) {
        id_qk[k] = make_idesc_mx(0u, 0u, MXA_BM, MXA_BN, k, k);
        id_pv[k] = make_idesc_mx(0u, 0u, MXA_BM, MXA_D, k, k) | (1u << 16);  // B (= V) MN-major
      }
      const uint64_t qdesc = make_smem_desc(smem_a + L::Q_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t pdesc = make_smem_desc(smem_a + L::P_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t kdesc0 = make_smem_desc(smem_a + L::KV_OFFSET, 16, 1024, SWIZZLE_128B);
      const uint64_t vdesc0 = make_smem_desc(smem_a + L::KV_OFFSET + L::TILE, L::TILE, 1024, SWIZZLE_128B);
      const uint64_t sfdesc0 = make_smem_desc(smem_a + L::SF_OFFSET, 16, 128, SWIZZLE_NONE);
      uint32_t kvs = 0, kvph = 0;  // ring position of the next K tile to multiply
      uint32_t vs = 0;             // ring position of the next V tile to multiply
      uint32_t sc = 0;             // S products issued so far (buffer = sc & 1)
      uint32_t pc = 0;             // P tiles consumed so far (tile n: buffer n & 1, barriers' phase n >> 1)
      uint32_t tcount = 0;
      bool ok = true;

      auto issue_qk = [&]() -> bool {
        if (!mbar_wait(&kv_full[kvs], kvph, status, WAIT_SMEM_FULL)) return false;
        tc_fence_after_sync();
        const uint32_t t_sfk = tmem_base + SFK_COL0 + (sc & 1) * 4;
        tmem_cp_32x128b_warpx4(t_sfk, sfdesc0 + (uint64_t)(((3 + 2 * kvs) * 512) >> 4));
        const uint64_t kd = kdesc0 + (uint64_t)((kvs * 2 * L::TILE) >> 4);
        const uint32_t d_s = tmem_base + S_COL0 + (sc & 1) * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_mxf8_ss(d_s, qdesc + 2 * k, kd + 2 * k, id_qk[k], tmem_base + SFQ_COL, t_sfk, k > 0 ? 1u : 0u);
        umma_commit(&s_full[sc & 1]);
        ++sc;
        if (++kvs == MXA_STAGES) {
          kvs = 0;
          kvph ^= 1;
        }
        return true;
      };

      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
        int bh, q0, nkv;
        mxa_tile(p, unit, bh, q0, nkv);
        if (!mbar_wait(q_full, tcount & 1, status, WAIT_ATTN)) break;
        // the previous tile's O must have been read out before PV(0) overwrites it
        if (!mbar_wait(o_free, (tcount & 1) ^ 1, status, WAIT_ATTN)) break;
        tc_fence_after_sync();
        tmem_cp_32x128b_warpx4(tmem_base + SFQ_COL, sfdesc0);
        if (!issue_qk()) break;
        for (int j = 0; j < nkv; ++j) {
          if (j + 1 < nkv) {
            if (!issue_qk()) {
              ok = false;
              break;
            }
          } else {
            umma_commit(q_empty);  // every S of this tile has been issued: Q may be replaced when they complete
          }
          // O += P(j) V(j): P tile number pc sits in buffer pc & 1
          const uint32_t pb = pc & 1;
          if (!mbar_wait(&p_full[pb], (pc >> 1) & 1, status, WAIT_ATTN)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t t_sfv = tmem_base + SFV_COL0 + pb * 4;
          const uint32_t t_sfp = tmem_base + SFP_COL0 + pb * 4;
          tmem_cp_32x128b_warpx4(t_sfp, sfdesc0 + (uint64_t)(((1 + pb) * 512) >> 4));
          tmem_cp_32x128b_warpx4(t_sfv, sfdesc0 + (uint64_t)(((4 + 2 * vs) * 512) >> 4));
          const uint64_t vd = vdesc0 + (uint64_t)((vs * 2 * L::TILE) >> 4);
          const uint64_t pd = pdesc + (uint64_t)((pb * L::TILE) >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_mxf8_ss(tmem_base + O_COL, pd + 2 * k, vd + (uint64_t)((k * 32 * 128) >> 4), id_pv[k],
                         t_sfp, t_sfv, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(&kv_empty[vs]);
          umma_commit(&pv_done[pb]);
          ++pc;
          if (++vs == MXA_STAGES) vs = 0;
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / epilogue
    // Two threads per query row: warps 4-7 take score columns 0-63 of their lane quarter's rows, warps 8-11 columns
    // 64-127 (a pass of one warp per scheduler over whole rows is bound by the length of that warp's instruction
    // stream; two warps per scheduler hide each other's latencies). The halves exchange their block maxima through
    // shared memory (a 64-thread named barrier per lane quarter) and keep partial row sums, added at the end.
    const int q = warp & 3;
    const int h = (warp - 4) >> 2;  // which half of the row
    const int row = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t t_o = tmem_base + lane_off + O_COL + h * 64;
    const float scale = p.scale_log2;
    const int s_kv = p.s_kv, s_q = p.s_q, causal = p.causal;
    uint8_t* const p_row0 = smem + L::P_OFFSET + row * 128;
    uint8_t* const p_scale0 = smem + L::SF_OFFSET + 512 + (row & 31) * 16 + (row >> 5) * 4 + h * 2;
    float* const xchg = reinterpret_cast<float*>(smem + L::XCHG_OFFSET);
    uint32_t sc = 0, tcount = 0;
    uint32_t pc = 0;  // P tiles written so far (buffer = pc & 1; the MMA side counts the same way)
    // the product with P tile n signals pv_done[n & 1], phase n >> 1
    auto wait_pv = [&](uint32_t n) -> bool { return mbar_wait(&pv_done[n & 1], (n >> 1) & 1, status, WAIT_ATTN); };
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory"); };
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
      int bh, q0, nkv;
      mxa_tile(p, unit, bh, q0, nkv);
      const int qrow = q0 + row;
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < nkv; ++j, ++sc) {
        if (!mbar_wait(&s_full[sc & 1], (sc >> 1) & 1, status, WAIT_ATTN)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_s = tmem_base + lane_off + S_COL0 + (sc & 1) * 128 + h * 64;
        uint32_t sv[64];
        tmem_ld_row32<0>(t_s, sv);
        tmem_ld_row32<32>(t_s + 32, sv);
        tmem_ld_wait();
        const int k0 = j * MXA_BN + h * 64;
        const bool need_mask = (j * MXA_BN + MXA_BN > s_kv) || (causal && (j * MXA_BN + MXA_BN - 1 > q0));
        const int limit = causal ? min(s_kv - 1, qrow) : (s_kv - 1);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (k0 + i > limit) sv[i] = 0xff800000u;
        }
        float bmax[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            mx0 = fmaxf(mx0, __uint_as_float(sv[b * 32 + i]));
            mx1 = fmaxf(mx1, __uint_as_float(sv[b * 32 + i + 1]));
          }
          bmax[b] = fmaxf(mx0, mx1);
        }
        // the row's block maximum over both halves
        float* const xs = xchg + (sc & 1) * 256;
        xs[h * 128 + row] = fmaxf(bmax[0], bmax[1]);
        pair_sync();
        const float m_blk = fmaxf(fmaxf(bmax[0], bmax[1]), xs[(h ^ 1) * 128 + row]) * scale;
        float alpha = 1.f;
        if (j == 0) {
          m = m_blk;
        } else if (m_blk - m > MXA_RESCALE_THRESHOLD) {
          alpha = fast_exp2(m - m_blk);
          m = m_blk;
        }
        // O may be rescaled only when the previous product is complete (rare: the lazy rescale), and this tile's P
        // buffer is free once the product before that one is (usually long since). Both halves of a row take the same
        // decisions (same maxima); each rescales its 64 columns of O.
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          if (!wait_pv(pc - 1)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 64; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_o + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32b_x32(t_o + c, v);
          }
          tmem_st_wait();
          tc_fence_before_sync();
        }
        if (pc >= 2 && !wait_pv(pc - 2)) {
          ok = false;
          break;
        }
        uint8_t* const p_row = p_row0 + (pc & 1) * L::TILE;
        uint16_t* const p_scale = reinterpret_cast<uint16_t*>(p_scale0 + (pc & 1) * 512);
        // p = exp2(s * scale - m); every 32 keys share the scale 2^ceil(log2(amax / 448)), where amax = exp2 of the
        // block's largest exponent (exp2 is monotonic: no second pass over p)
        uint32_t scale_word = 0;
        const uint64_t scale2 = pack2(scale, scale), negm2 = pack2(-m, -m);
        uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const float amax = fast_exp2(fmaf(bmax[b], scale, -m));
          const uint32_t bits = (__float_as_uint(amax * (1.f / 448.f)) + 0x007FFFFFu) & 0x7F800000u;
          const float inv = bits == 0u ? 0.f : __uint_as_float(0x7F000000u - bits);  // 2^-(e - 127), exact
          const uint64_t inv2 = pack2(inv, inv);
          scale_word |= (bits >> 23) << (8 * b);
#pragma unroll
          for (int c = 0; c < 2; ++c) {  // two 16-byte chunks per block
            uint32_t w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint16_t hh[2];
#pragma unroll
              for (int t = 0; t < 2; ++t) {  // packed f32x2 arithmetic: one instruction per pair
                const int i = b * 32 + c * 16 + u * 4 + t * 2;
                const uint64_t x = fma2(pack2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, negm2);
                float x0, x1;
                unpack2(x, x0, x1);
                const uint64_t e = pack2(fast_exp2(x0), fast_exp2(x1));
                sum2 = add2(sum2, e);
                float q0f, q1f;
                unpack2(mul2(e, inv2), q0f, q1f);
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hh[t]) : "f"(q1f), "f"(q0f));
              }
              w[u] = (uint32_t)hh[0] | ((uint32_t)hh[1] << 16);
            }
            const int chunk = h * 4 + b * 2 + c;
            *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        float sum_lo, sum_hi;
        unpack2(sum2, sum_lo, sum_hi);
        *p_scale = (uint16_t)scale_word;
        l += sum_lo + sum_hi;
        fence_proxy_async_smem();
        mbar_arrive(&p_full[pc & 1]);
        ++pc;
      }
      if (!ok) break;
      // ---- epilogue: the last PV, then O / l as bf16 and the base-2 log-sum-exp; the halves add their row sums
      if (!wait_pv(pc - 1)) break;
      tc_fence_after_sync();
      float* const xs = xchg + (tcount & 1) * 256;
      pair_sync();  // the pair has left the last block's exchange
      xs[h * 128 + row] = l;
      pair_sync();
      l += xs[(h ^ 1) * 128 + row];
      pair_sync();  // both have read: the exchange area may be written again
      const float inv_l = 1.f / l;
      const bool valid = qrow < s_q;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + ((size_t)bh * s_q + qrow) * MXA_D + h * 64;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_o + c, v);
        tmem_ld_wait();
        if (valid) {
          uint32_t w[16];
#pragma unroll
          for (int u = 0; u < 16; ++u)
            w[u] = pack_bf16x2(__uint_as_float(v[2 * u]) * inv_l, __uint_as_float(v[2 * u + 1]) * inv_l);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(orow + c)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(o_free);
      if (valid && h == 0 && p.lse) p.lse[(size_t)bh * s_q + qrow] = m + log2f(l);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_attention_mxfp8_fwd(const tb200_attention_mxfp8_args* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->o || !a->q_scale || !a->k_scale || !a->v_scale) return TB200_ERR_BAD_ARG;
  if (a->batch < 0 || a->heads < 0 || a->seq_q < 0 || a->seq_kv < 0) return TB200_ERR_BAD_ARG;
  if (a->head_dim != MXA_D) return TB200_ERR_UNSUPPORTED;
  if ((a->seq_q % 128) || (a->seq_kv % 128)) return TB200_ERR_UNSUPPORTED;  // whole scale atoms
  if (a->causal && a->seq_q != a->seq_kv) return TB200_ERR_UNSUPPORTED;
  if (!(a->sm_scale > 0.f)) return TB200_ERR_BAD_ARG;
  const long long bh = (long long)a->batch * a->heads;
  if (bh == 0 || a->seq_q == 0) return TB200_OK;
  if (a->seq_kv == 0) return TB200_ERR_BAD_ARG;
  if (bh > INT32_MAX || a->seq_q > (1 << 30) || a->seq_kv > (1 << 30)) return TB200_ERR_UNSUPPORTED;
  const void* ptrs[7] = {a->q, a->k, a->v, a->o, a->q_scale, a->k_scale, a->v_scale};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  MxAttnParams p;
  memset(&p, 0, sizeof(p));
  const uint32_t box[3] = {128, 128, 1};
  {
    const uint64_t dims[3] = {(uint64_t)MXA_D, (uint64_t)a->seq_q, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)MXA_D, (uint64_t)a->seq_q * MXA_D};
    int rc = encode_tmap(&p.tmq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)MXA_D, (uint64_t)a->seq_kv, (uint64_t)bh};
    const uint64_t strides[2] = {(uint64_t)MXA_D, (uint64_t)a->seq_kv * MXA_D};
    int rc = encode_tmap(&p.tmk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap(&p.tmv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.sfq = static_cast<const uint8_t*>(a->q_scale);
  p.sfk = static_cast<const uint8_t*>(a->k_scale);
  p.sfv = static_cast<const uint8_t*>(a->v_scale);
  p.o = a->o;
  p.lse = a->lse;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.bh = (int)bh;
  p.s_q = (int)a->seq_q;
  p.s_kv = (int)a->seq_kv;
  p.q_tiles = (int)(a->seq_q / MXA_BM);
  p.units = p.q_tiles * p.bh;
  p.causal = a->causal ? 1 : 0;
  // non-causal: head-major order (the same speed - 1023 against 1017 TFLOP/s at [4, 32, 8192, 128] - with each head's
  // K and V read from HBM once instead of once per query tile); causal: longest tiles first (976 against 909)
  p.head_major = a->causal ? 0 : 1;
  p.scale_log2 = a->sm_scale * 1.4426950408889634f;
  auto kfn = attention_mxfp8_fwd_kernel;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, MxAttnSmem::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  const int grid = p.units < sms ? p.units : sms;
  kfn<<<grid, MXA_THREADS, MxAttnSmem::TOTAL, stream>>>(p);
  return cuda_err(cudaGetLastError());
}
