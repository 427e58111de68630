// Dense GEMM for sm_100a: persistent, warp-specialised, TMA -> shared-memory ring ->
// tcgen05.mma with the accumulator double-buffered in tensor memory -> epilogue warps.
//
// Roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane; the warp
// also owns the TMEM allocation), warps 2..5 = epilogue (each reads its own 32-lane quarter of
// TMEM). K step = 128 bytes of K per operand row (64 16-bit or 128 8-bit elements) = 4 MMAs.
// The same kernel serves bf16/fp16 (kind::f16) and e4m3/e5m2 (kind::f8f6f4).
//
// Two tilings:
//   single CTA : 128 x BN tile per CTA, BN in {64, 128, 256}.
//   CTA pair   : a 2-CTA cluster shares one 256 x 256 tile. CTA r loads A rows [m0+128r, +128)
//                and B rows (N) [n0+128r, +128); the leader (rank 0) issues
//                tcgen05.mma.cta_group::2 with M = 256, which reads A from each CTA's own shared
//                memory and the two halves of B from both, and leaves rows 128r..128r+127 of the
//                accumulator in CTA r's tensor memory. Per CTA a K step lands 32 KB instead of
//                48 KB: a step's traffic through the 128 B/clk shared-memory port (TMA writes plus
//                the MMAs' operand reads) drops from 96 KB (750 cycles per 512 of MMA) to 80 KB.
//                Signalling: TMA bytes of both CTAs count on the leader's `full` barrier; the
//                leader issues one tcgen05.commit per CTA onto that CTA's `empty` / `tfull` barrier
//                (two plain commits, no multicast); epilogue warps of both CTAs arrive on the
//                leader's `tempty`.
//
//   wide pair  : the same with a 256 x 512 tile: each CTA stages 128 A rows and 256 B rows per K step, the
//                leader issues two N = 256 MMAs per K sub-step into the two halves of a single 512-column
//                accumulator (all of tensor memory: there is no second accumulator to overlap the epilogue
//                with, so the halves are handed over separately and the first / last K steps of a tile work
//                on one half while the other is drained). A is staged once for 512 columns: per 1024 MMA cycles a
//                CTA's port carries 48 KB of TMA writes + 96 KB of operand reads at most, against
//                2 x (32 + 48) KB for two 256 x 256 tiles - the port stops being the limit (tensor pipe
//                active 85 % -> measured below), and L2 -> SM traffic per flop drops by a quarter.
//
// Split K, two forms. Few tiles and a long K (one row of tiles: M <= 128 against N = K = 8192) leave most SMs
// idle and the B stream latency-bound, so K is cut into split_k ranges handled by different CTAs.
//   in-cluster : when all of a tile's splits fit one wave (tiles x split_k <= SMs, split_k <= 8) they are launched as
//                one thread-block cluster. Each CTA leaves its fp32 partial tile in its own shared memory (the
//                operand ring is free by then), the cluster synchronises, and CTA r sums columns
//                [r BN / split_k, (r + 1) BN / split_k) of all partials through distributed shared memory, in
//                rank order (deterministic), converts and stores them. One launch, no workspace, no second pass
//                over HBM (the reference reduces through a workspace: _reduce_k_kernel,
//                third_party/tlx/tutorials/blackwell_gemm_ws.py:1098-1122).
//   workspace  : otherwise fp32 partials go to a caller workspace and splitk_reduce_kernel sums them.
//
// The issue loops are kept lean on purpose: measured on B200, tcgen05.mma issue blocks the issuing
// thread until the tensor pipe accepts the instruction, so every other instruction in the MMA
// thread's loop is exposed tensor-pipe idle time. All loop-invariant parameters are copied to
// registers first (inline asm with a memory clobber otherwise forces re-loads from the parameter
// bank), descriptors advance by integer adds, stage/phase are running counters, and the commit
// and the wait of each K step are placed between its MMAs.
//
// Counterpart in the reference: matmul_kernel_tma_ws_blackwell,
// third_party/tlx/tutorials/blackwell_gemm_ws.py:1168-1483 (producer :961-1088, MMA :840-957,
// epilogue :680-836) and the tensorwise path of blackwell_scaled_mm_ws.py:51-378.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int BM = 128;
static constexpr int STAGE_K_BYTES = 128;  // bytes of K per operand row per stage (one swizzle atom)
static constexpr int GEMM_THREADS = 192;

struct OperandGeom {
  uint32_t boxes;       // TMA copies per stage
  uint32_t box_bytes;   // bytes each copy lands
  uint32_t box_mn;      // rows (K-major) or MN elements (MN-major) covered by one box
  uint32_t lbo, sbo;    // descriptor leading / stride byte offsets
  uint32_t kstep;       // bytes added to the descriptor start address per MMA K step
  uint32_t mn_major;    // 0: K-major tile, 1: MN-major tile
};

struct GemmParams {
  CUtensorMap tma;
  CUtensorMap tmb;
  CUtensorMap tmc;  // output as 64-column x 32-row boxes (wide tile, 16-bit output); valid when c_tma != 0
  void* c;
  float* ws;
  const float* scale_a;
  const float* scale_b;
  int* status;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n, units;  // units = tiles_m * tiles_n * split_k
  int k_blocks, split_k, kb_per_split;
  int bk_elems;  // K elements per stage
  int group_m;
  int out_mode;  // 0 bf16, 1 fp16, 2 fp32 to c, 3 fp32 partial to ws
  int scale_mode;  // 0: scale_a / scale_b are scalars; 1: per-row (M) and per-column (N) vectors
  int c_tma;       // 1: the wide kernel's epilogue stores through tmc
  int cluster_k;   // > 1: the split_k CTAs of a tile form a cluster and sum their partials through shared memory
  uint32_t idesc;
  OperandGeom ga, gb;
};

// BNC = B rows (N) staged per CTA; the tile is 128 x BNC (single) or 256 x 256 (pair, BNC = 128).
template <int BNC, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * STAGE_K_BYTES;
  static constexpr int B_BYTES = BNC * STAGE_K_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
  // wide tile: per epilogue warp two 4 KB staging buffers (32 rows x 128 bytes) for TMA stores, 1 KB past the barriers
  static constexpr int EPI_OFFSET = BAR_OFFSET + 1024;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;
  static constexpr int TOTAL_WIDE = EPI_OFFSET + EPI_BYTES + 1024;
};

template <bool PAIR, bool F8>
__device__ __forceinline__ void issue_mma(uint32_t tmem_d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t accum) {
  if constexpr (PAIR) {
    if constexpr (F8)
      umma_f8_ss_pair(tmem_d, ad, bd, idesc, accum);
    else
      umma_f16_ss_pair(tmem_d, ad, bd, idesc, accum);
  } else {
    if constexpr (F8)
      umma_f8_ss(tmem_d, ad, bd, idesc, accum);
    else
      umma_f16_ss(tmem_d, ad, bd, idesc, accum);
  }
}

template <int BNC, int STAGES, bool PAIR, bool F8>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  using L = GemmSmem<BNC, STAGES>;
  constexpr int BN = PAIR ? 2 * BNC : BNC;    // accumulator columns per tile
  constexpr int TILE_M = PAIR ? 256 : BM;     // output rows per scheduling unit
  constexpr bool WIDE = PAIR && BNC == 256;   // 256 x 512 tile: two N = 256 MMAs per K step, one accumulator
  constexpr uint32_t NACC = WIDE ? 1 : 2;     // accumulators in tensor memory
  constexpr uint32_t TMEM_COLS = (NACC * BN < 32) ? 32 : NACC * BN;
  // descriptor offset (16-byte units) of the second 128 B rows inside a CTA's staged B tile: 16 KB in both layouts
  constexpr uint64_t B_HALF = (128 * STAGE_K_BYTES) >> 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  // split-K: the reduction pass behind this grid may be launched now (it waits for this grid's completion itself)
  if (p.out_mode == 3) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma);
    tma_prefetch_desc(&p.tmb);
    if (WIDE && p.c_tma) tma_prefetch_desc(&p.tmc);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], PAIR ? 8 : 4);
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // loop-invariant scheduling parameters in registers
  const int units = p.units, split_k = p.split_k, group_m = p.group_m, tiles_m = p.tiles_m, tiles_n = p.tiles_n;
  const int k_blocks = p.k_blocks, kb_per_split = p.kb_per_split;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      const int bk_elems = p.bk_elems;
      const uint32_t a_boxes = p.ga.boxes, a_box_bytes = p.ga.box_bytes, a_box_mn = p.ga.box_mn, a_mn = p.ga.mn_major;
      const uint32_t b_boxes = p.gb.boxes, b_box_bytes = p.gb.box_bytes, b_box_mn = p.gb.box_mn, b_mn = p.gb.mn_major;
      const uint32_t leader_full = PAIR ? mapa_shared(full_a, 0) : full_a;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = worker; unit < units && ok; unit += num_workers) {
        const TileCoord t = unit_to_tile(unit, split_k, group_m, tiles_m, tiles_n);
        const int m0 = t.pid_m * TILE_M + (int)rank * BM;
        const int n0 = t.pid_n * BN + (int)rank * BNC * (PAIR ? 1 : 0);
        const int kb0 = t.ks * kb_per_split;
        const int kb1 = min(k_blocks, kb0 + kb_per_split);
        int kx = kb0 * bk_elems;
        for (int kb = kb0; kb < kb1; ++kb, kx += bk_elems) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if constexpr (PAIR) {
            // the leader's barrier counts both CTAs' bytes
            if (rank == 0) mbar_expect_tx_a(full_a + s * 8, 2 * L::STAGE_BYTES);
          } else {
            mbar_expect_tx_a(full_a + s * 8, L::STAGE_BYTES);
          }
          const uint32_t bar = leader_full + s * 8;
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          const uint32_t sb = sa + L::A_BYTES;
          for (uint32_t i = 0; i < a_boxes; ++i) {
            const int mn = m0 + (int)(i * a_box_mn);
            if constexpr (PAIR)
              tma_load_2d_pair(sa + i * a_box_bytes, &p.tma, bar, a_mn ? mn : kx, a_mn ? kx : mn, pol);
            else
              tma_load_2d_a(sa + i * a_box_bytes, &p.tma, bar, a_mn ? mn : kx, a_mn ? kx : mn, pol);
          }
          for (uint32_t i = 0; i < b_boxes; ++i) {
            const int mn = n0 + (int)(i * b_box_mn);
            if constexpr (PAIR)
              tma_load_2d_pair(sb + i * b_box_bytes, &p.tmb, bar, b_mn ? mn : kx, b_mn ? kx : mn, pol);
            else
              tma_load_2d_a(sb + i * b_box_bytes, &p.tmb, bar, b_mn ? mn : kx, b_mn ? kx : mn, pol);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = p.idesc;
      const uint64_t ak = (uint64_t)(p.ga.kstep >> 4), bk = (uint64_t)(p.gb.kstep >> 4);
      const uint64_t adesc0 = make_smem_desc(smem_a, p.ga.lbo, p.ga.sbo, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, p.gb.lbo, p.gb.sbo, SWIZZLE_128B);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      const uint32_t tfull_peer = PAIR ? mapa_shared(tfull_a, 1) : 0u;
      // shared::cluster address of the peer's copy of a barrier = own address + peer_delta
      const uint32_t peer_delta = PAIR ? (mapa_shared(empty_a, 1) - empty_a) : 0u;
      uint32_t s = 0, ph = 0, tcount = 0;
      bool ok = true;
      for (int unit = worker; unit < units && ok; unit += num_workers, ++tcount) {
        const TileCoord t = unit_to_tile(unit, split_k, group_m, tiles_m, tiles_n);
        const int kb0 = t.ks * kb_per_split;
        const int nkb = min(k_blocks, kb0 + kb_per_split) - kb0;
        if constexpr (WIDE) {
          // One 512-column accumulator, handed over in two 256-column halves (tfull / tempty index = half) so
          // that the drain of one half overlaps MMAs on the other: the first HEAD K steps of a tile run on half
          // 0 alone while the epilogue still drains half 1 of the previous tile, and the last TAIL steps finish
          // half 0 first so that its drain starts while half 1 is completed. A stage is released when both halves
          // have read it, so at most STAGES - 1 steps are held back.
          const uint32_t tph = tcount & 1;
          const int head = nkb < STAGES - 1 ? nkb : STAGES - 1;
          const int tail = (nkb - head) < STAGES - 1 ? (nkb - head) : STAGES - 1;
          auto half_step = [&](uint32_t st, uint32_t h, uint32_t accumulate) {
            const uint64_t ad = adesc0 + (uint64_t)(st * (L::STAGE_BYTES >> 4));
            const uint64_t bd = bdesc0 + (uint64_t)(st * (L::STAGE_BYTES >> 4)) + h * B_HALF;
            const uint32_t d = tmem_base + h * 256;
            issue_mma<PAIR, F8>(d, ad, bd, idesc, accumulate);
            issue_mma<PAIR, F8>(d, ad + ak, bd + bk, idesc, 1u);
            issue_mma<PAIR, F8>(d, ad + 2 * ak, bd + 2 * bk, idesc, 1u);
            issue_mma<PAIR, F8>(d, ad + 3 * ak, bd + 3 * bk, idesc, 1u);
          };
          auto release = [&](uint32_t st) {
            umma_commit_pair(empty_a + st * 8);
            umma_commit_pair(empty_a + st * 8 + peer_delta);
          };
          auto wait_full = [&]() {
            if (!mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) return false;
            tc_fence_after_sync();
            return true;
          };
          auto advance = [&](uint32_t& st, uint32_t& phase) {
            if (++st == STAGES) {
              st = 0;
              phase ^= 1;
            }
          };
          if (!mbar_wait_a(tempty_a, tph ^ 1, status, WAIT_TMEM_EMPTY)) break;
          tc_fence_after_sync();
          uint32_t s_held = s, ph_unused = 0;
          for (int i = 0; i < head && ok; ++i) {
            ok = wait_full();
            if (ok) {
              half_step(s, 0, i == 0 ? 0u : 1u);
              advance(s, ph);
            }
          }
          if (!ok) break;
          if (!mbar_wait_a(tempty_a + 8, tph ^ 1, status, WAIT_TMEM_EMPTY)) break;
          tc_fence_after_sync();
          for (int i = 0; i < head; ++i) {
            half_step(s_held, 1, i == 0 ? 0u : 1u);
            release(s_held);
            advance(s_held, ph_unused);
          }
          for (int i = head; i < nkb - tail && ok; ++i) {
            ok = wait_full();
            if (ok) {
              const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
              const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                issue_mma<PAIR, F8>(tmem_base, ad + j * ak, bd + j * bk, idesc, 1u);
                issue_mma<PAIR, F8>(tmem_base + 256, ad + j * ak, bd + j * bk + B_HALF, idesc, 1u);
              }
              release(s);
              advance(s, ph);
            }
          }
          if (!ok) break;
          s_held = s;
          for (int i = 0; i < tail && ok; ++i) {
            ok = wait_full();
            if (ok) {
              half_step(s, 0, 1u);
              advance(s, ph);
            }
          }
          if (!ok) break;
          umma_commit_pair(tfull_a);
          umma_commit_pair(tfull_peer);
          for (int i = 0; i < tail; ++i) {
            half_step(s_held, 1, 1u);
            release(s_held);
            advance(s_held, ph_unused);
          }
          umma_commit_pair(tfull_a + 8);
          umma_commit_pair(tfull_peer + 8);
          continue;
        }
        const uint32_t acc = tcount % NACC;
        const uint32_t aph = (tcount / NACC) & 1;
        if (!mbar_wait_a(tempty_a + acc * 8, aph ^ 1, status, WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        auto mma_step = [&](uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
          issue_mma<PAIR, F8>(tmem_d, a_desc, b_desc, idesc, accumulate);
        };
        // Loop shape: every non-MMA instruction sits between two MMAs of the same K step, where it
        // overlaps with tensor-pipe work already queued: the commit that frees the previous stage
        // comes after this step's first MMA, the wait for the next stage after the second.
        if (!mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t accum = 0;
        uint32_t prev_empty = 0;  // barrier address of the stage whose release is still owed
        for (int i = 0; i < nkb; ++i) {
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          mma_step(ad, bd, accum);
          accum = 1u;
          if (prev_empty) {
            if constexpr (PAIR) {
              umma_commit_pair(prev_empty);
              umma_commit_pair(prev_empty + peer_delta);
            } else {
              umma_commit_a(prev_empty);
            }
          }
          prev_empty = empty_a + s * 8;
          mma_step(ad + ak, bd + bk, 1u);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
          if (i + 1 < nkb) {
            if (!mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          mma_step(ad + 2 * ak, bd + 2 * bk, 1u);
          mma_step(ad + 3 * ak, bd + 3 * bk, 1u);
        }
        if (ok) {
          if constexpr (PAIR) {
            umma_commit_pair(prev_empty);
            umma_commit_pair(prev_empty + peer_delta);
            umma_commit_pair(tfull_a + acc * 8);
            umma_commit_pair(tfull_peer + acc * 8);
          } else {
            umma_commit_a(prev_empty);
            umma_commit_a(tfull_a + acc * 8);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const bool rowwise = p.scale_mode == 1;
    float alpha = 1.0f;
    if (!rowwise) {
      if (p.scale_a) alpha *= __ldg(p.scale_a);
      if (p.scale_b) alpha *= __ldg(p.scale_b);
    }
    const float* const row_scale = rowwise ? p.scale_a : nullptr;
    const float* const col_scale = rowwise ? p.scale_b : nullptr;
    void* const c = p.c;
    float* const ws = p.ws;
    const long long ldc = p.ldc;
    const int m = p.m, n = p.n, out_mode = p.out_mode;
    const uint32_t tempty_leader = PAIR ? mapa_shared(smem_u32(tempty), 0) : smem_u32(tempty);
    [[maybe_unused]] const bool use_tma = WIDE && p.c_tma != 0;
    [[maybe_unused]] const uint32_t stage_base = smem_a + L::EPI_OFFSET + (uint32_t)q * 8192;
    [[maybe_unused]] uint32_t slab = 0;
    [[maybe_unused]] const uint64_t store_pol = policy_evict_first();
    uint32_t tcount = 0;
    bool ok = true;
    for (int unit = worker; unit < units && ok; unit += num_workers, ++tcount) {
      const TileCoord t = unit_to_tile(unit, split_k, group_m, tiles_m, tiles_n);
      const int m0 = t.pid_m * TILE_M + (int)rank * BM, n0 = t.pid_n * BN;
      const int row = m0 + q * 32 + lane;
      if constexpr (WIDE) {
        // the two 256-column halves arrive and are handed back separately (barrier index = half)
        const uint32_t tph = tcount & 1;
        if (row_scale) alpha = row < m ? __ldg(row_scale + row) : 0.f;
        for (int h = 0; h < 2 && ok; ++h) {
          if (!mbar_wait(&tfull[h], tph, status, WAIT_TMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + h * 256;
          // accumulator columns [128 j, 128 j + 128) of the tile hold output columns of the B rows staged by CTA
          // (j & 1) and read by MMA (j >> 1) = half: CTA r stages rows n0 + 256 r .. + 255, half h takes rows
          // 128 h .. 128 h + 127 of each
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(taddr, v0);
          if (use_tma) {
            // 16-bit output through shared memory: 64 columns of the warp's 32 rows (128 bytes per row, 128-byte
            // swizzle) per TMA store, two staging buffers per warp. The store engine writes whole lines and clips
            // at the matrix edge; per-thread stores here wrote one 32-byte sector per thread and instruction, and
            // all CTAs drain at the same time: that cost 3000 cycles per 256 columns.
#pragma unroll 1
            for (int cc = 0; cc < 256; cc += 64) {
              const int gc = n0 + (cc >> 7) * 256 + h * 128 + (cc & 127);
              const uint32_t buf = stage_base + (uint32_t)(slab & 1) * 4096;
              ++slab;
              if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this buffer has finished
              __syncwarp();
              tmem_ld_wait();
              tmem_ld_32x32b_x32(taddr + cc + 32, v1);
              stage_chunk(buf, lane, 0, v0, gc, out_mode, alpha, col_scale, n);
              tmem_ld_wait();
              if (cc + 64 < 256) tmem_ld_32x32b_x32(taddr + cc + 64, v0);
              stage_chunk(buf, lane, 4, v1, gc + 32, out_mode, alpha, col_scale, n);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (gc < n && m0 + q * 32 < m) tma_store_2d_hint(&p.tmc, buf, gc, m0 + q * 32, store_pol);  // edges are clipped
                bulk_commit_group();
              }
            }
          } else {
#pragma unroll 1
            for (int cc = 0; cc < 256; cc += 64) {
              const int gc = n0 + (cc >> 7) * 256 + h * 128 + (cc & 127);
              tmem_ld_wait();
              tmem_ld_32x32b_x32(taddr + cc + 32, v1);
              store_chunk(c, ws, ldc, m, n, out_mode, v0, row, gc, t.ks, alpha, col_scale);
              tmem_ld_wait();
              if (cc + 64 < 256) tmem_ld_32x32b_x32(taddr + cc + 64, v0);
              store_chunk(c, ws, ldc, m, n, out_mode, v1, row, gc + 32, t.ks, alpha, col_scale);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader + h * 8);
        }
        continue;
      }
      const uint32_t acc = tcount % NACC;
      const uint32_t aph = (tcount / NACC) & 1;
      if (!mbar_wait(&tfull[acc], aph, status, WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      if constexpr (!PAIR) {
        if (p.cluster_k > 1) {
          // in-cluster split K: leave this CTA's partial tile in shared memory, column-major ([column][row], fp32),
          // so that lanes (= rows) touch consecutive words here and in the remote reads of the reduction below
          const uint32_t red = smem_a + (uint32_t)(q * 32 + lane) * 4;
#pragma unroll 1
          for (int cc = 0; cc < BN; cc += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(taddr + cc, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(red + (uint32_t)(cc + j) * (BM * 4)), "r"(v[j]) : "memory");
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_a(tempty_leader + acc * 8);
          continue;
        }
      }
      if (row_scale) alpha = row < m ? __ldg(row_scale + row) : 0.f;
      auto out_col = [&](int cc) { return n0 + cc; };
      if constexpr (BN >= 64) {
        // two chunks in flight: the next tensor-memory load runs while this chunk is converted and stored
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(taddr, v0);
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 64) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(taddr + cc + 32, v1);
          store_chunk(c, ws, ldc, m, n, out_mode, v0, row, out_col(cc), t.ks, alpha, col_scale);
          tmem_ld_wait();
          if (cc + 64 < BN) tmem_ld_32x32b_x32(taddr + cc + 64, v0);
          store_chunk(c, ws, ldc, m, n, out_mode, v1, row, out_col(cc + 32), t.ks, alpha, col_scale);
        }
      } else {
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + cc, v);
          tmem_ld_wait();
          store_chunk(c, ws, ldc, m, n, out_mode, v, row, out_col(cc), t.ks, alpha, col_scale);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR)
          mbar_arrive_cluster(tempty_leader + acc * 8);
        else
          mbar_arrive_a(tempty_leader + acc * 8);
      }
    }
  }

  if constexpr (WIDE) {
    if (warp >= 2 && lane == 0) bulk_wait_group<0>();  // this thread's TMA stores have completed
  }
  if constexpr (!PAIR) {
    if (p.cluster_k > 1) {
      // ---- in-cluster split-K reduction: every CTA of the cluster holds the partial of the same tile
      __syncwarp();
      cluster_sync_all();  // all partials are in shared memory (the role loops above leave no thread behind)
      if (warp >= 2 && worker < units) {
        const int q = warp & 3;
        const int S = p.cluster_k;
        const TileCoord t = unit_to_tile(worker, split_k, group_m, tiles_m, tiles_n);
        const int row = t.pid_m * BM + q * 32 + lane;
        const int cols_per = BN / S;                      // a multiple of 32 (checked on the host)
        const int c_first = (int)cluster_ctarank() * cols_per;
        const bool rowwise = p.scale_mode == 1;
        float alpha = 1.0f;
        if (rowwise) {
          alpha = row < p.m ? __ldg(p.scale_a + row) : 0.f;
        } else {
          if (p.scale_a) alpha *= __ldg(p.scale_a);
          if (p.scale_b) alpha *= __ldg(p.scale_b);
        }
        const uint32_t own = smem_a + (uint32_t)(q * 32 + lane) * 4;
        uint32_t remote[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) remote[r] = r < S ? mapa_shared(own, (uint32_t)r) : 0u;
#pragma unroll 1
        for (int cc = c_first; cc < c_first + cols_per; cc += 32) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
#pragma unroll 1
          for (int r = 0; r < S; ++r) {   // rank order: the sum does not depend on which CTA finished first
            const uint32_t base = remote[r] + (uint32_t)cc * (BM * 4);
            float x[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x[j]) : "r"(base + (uint32_t)j * (BM * 4)) : "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + x[j]);
          }
          store_chunk(p.c, nullptr, p.ldc, p.m, p.n, p.out_mode, v, row, t.pid_n * BN + cc, 0, alpha,
                      rowwise ? p.scale_b : nullptr);
        }
      }
      __syncwarp();
      cluster_sync_all();  // nobody leaves (and frees its shared memory) while a peer may still read it
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR)
      tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else
      tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// C[m,n] = sum_s ws[s,m,n] (fp32) -> out dtype. One thread per 4 consecutive columns.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ c, int m, int n, long long ldc,
                                     int split_k, int out_mode) {
  // launched with programmatic stream serialization right behind the GEMM that writes ws: its blocks may be resident
  // before that grid has finished, and wait here until it has (and its writes are visible)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long n4 = (n + 3) / 4;
  const long long total = (long long)m * n4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / n4);
    const int col = (int)(i - (long long)row * n4) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int cnt = min(4, n - col);
    const bool vec = (cnt == 4) && ((n & 3) == 0);
    for (int s = 0; s < split_k; ++s) {
      const float* src = ws + ((long long)s * m + row) * (long long)n + col;
      if (vec) {
        float4 v = *reinterpret_cast<const float4*>(src);
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      } else {
        for (int j = 0; j < cnt; ++j) acc[j] += src[j];
      }
    }
    for (int j = 0; j < cnt; ++j) {
      const long long o = (long long)row * ldc + col + j;
      if (out_mode == 0)
        reinterpret_cast<__nv_bfloat16*>(c)[o] = __float2bfloat16_rn(acc[j]);
      else if (out_mode == 1)
        reinterpret_cast<__half*>(c)[o] = __float2half_rn(acc[j]);
      else
        reinterpret_cast<float*>(c)[o] = acc[j];
    }
  }
}

// ------------------------------------------------------------------------------- host

struct GemmPlan {
  int pair;  // 1: CTA-pair kernel, 256 x 256 tile per cluster; 2: 256 x 512 tile per cluster
  int bn;
  int cluster_reduce;  // 1: the split_k CTAs of a tile form a cluster and reduce through shared memory (no workspace)
  int split_k;
  int kb_per_split;
  int k_blocks;
  int tiles_m, tiles_n;
};

static int elem_bytes(int dtype) {
  switch (dtype) {
    case TB200_BF16:
    case TB200_F16: return 2;
    case TB200_E4M3:
    case TB200_E5M2: return 1;
    default: return 0;
  }
}

static bool plan_gemm(const tb200_gemm_args* a, int sms, GemmPlan* plan) {
  const int eb = elem_bytes(a->in_dtype);
  if (eb == 0) return false;
  const int bk = STAGE_K_BYTES / eb;
  const long long kb = (a->k + bk - 1) / bk;
  const long long tm = (a->m + BM - 1) / BM;
  int bn = a->block_n;
  int pair = 0;
  long long tm_eff = tm;
  if (bn == 512) {
    pair = 1;
    bn = 256;
  } else if (bn == 1024) {
    pair = 2;
    bn = 512;
  } else if (bn == 0) {
    // Estimated time = waves x per-tile cost; one SM handles a 128 x bn tile in ~(bn + 48) units.
    long long best = -1;
    const int cands[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i) {
      const int cbn = cands[i];
      const long long tiles = tm * ((a->n + cbn - 1) / cbn);
      const long long waves = (tiles + sms - 1) / sms;
      const long long cost = waves * (cbn + 48) * 4;
      if (best < 0 || cost < best) {
        best = cost;
        bn = cbn;
      }
    }
    // One row of tiles and a long K: such a GEMM streams B at the rate (stages in flight) / (load latency), so a CTA
    // per 128 x 64 tile walking all of K (one short wave) is slower than 128-wide tiles with K split in two or
    // more, although that adds the partial-sum pass (M = 128, N = K = 8192: 46 us against 31 + 6).
    // (The B stream of this shape is bound by the loads in flight, not by DRAM page locality: a producer that waited
    // for two or three free stages and issued their loads back to back - consecutive 128-byte pieces of the same rows
    // close in time - measured 43.5 / 45.5 us against 35.5.)
    if (tm == 1 && kb >= 32 && a->split_k <= 0) {
      const long long t128 = (a->n + 127) / 128;
      if (t128 * 2 <= sms) bn = 128;
    }
    // CTA pair: two SMs share a 256 x 256 tile; each still computes 128 x 256 but stages a third
    // less data per K step, which is worth ~25% once the grid is full.
    if (a->m > BM && sms >= 2) {
      const long long tiles2 = ((a->m + 255) / 256) * ((a->n + 255) / 256);
      const long long waves2 = (tiles2 + sms / 2 - 1) / (sms / 2);
      const long long cost2 = waves2 * (256 + 48) * 3;
      if (cost2 <= best) {
        pair = 1;
        bn = 256;
        best = cost2;
      }
      // 256 x 512 per pair: twice the tile at ~88 % of twice the cost (measured at 8192^3), plus an epilogue that
      // is only partly overlapped (~9000 cycles a tile against 1024 per K step): worth it when the coarser tiles
      // still fill the waves and K is long (measured: ahead from 48 K steps on, behind at 32)
      const long long tiles3 = ((a->m + 255) / 256) * ((a->n + 511) / 512);
      const long long waves3 = (tiles3 + sms / 2 - 1) / (sms / 2);
      const long long cost3 = waves3 * (512 + 24) * 3 * 88 / 100;
      if (cost3 < best && kb >= 48) {
        pair = 2;
        bn = 512;
      }
    }
  }
  if (bn != 64 && bn != 128 && bn != 256 && !(pair == 2 && bn == 512)) return false;
  if (pair) tm_eff = (a->m + 255) / 256;
  const long long tn = (a->n + bn - 1) / bn;
  const long long tiles = tm_eff * tn * (pair ? 2 : 1);
  long long split = a->split_k;
  if (split <= 0) {
    split = 1;
    // Few tiles and a long K: partition K so most SMs have work (each part keeps >= 8 K blocks).
    if (tiles * 2 <= sms && kb >= 16) {
      split = sms / tiles;
      if (split > kb / 8) split = kb / 8;
      if (split > 16) split = 16;
      if (split < 1) split = 1;
    }
  }
  if (split > kb) split = kb > 0 ? kb : 1;
  long long per = kb > 0 ? (kb + split - 1) / split : 0;
  if (per > 0) split = (kb + per - 1) / per;
  // all splits of every tile resident at once, as clusters of split CTAs (power of two, at most 8, and at least 32
  // output columns per CTA in the reduction): the partial sums never leave the SMs
  plan->cluster_reduce = (!pair && split > 1 && split <= 8 && (split & (split - 1)) == 0 && tiles * split <= sms &&
                          bn / split >= 32) ? 1 : 0;
  plan->pair = pair;
  plan->bn = bn;
  plan->split_k = (int)split;
  plan->kb_per_split = (int)per;
  plan->k_blocks = (int)kb;
  plan->tiles_m = (int)tm_eff;
  plan->tiles_n = (int)tn;
  return true;
}

template <int BNC, int STAGES, bool PAIR, bool F8>
static int launch_one(const GemmParams& p, int grid, cudaStream_t stream) {
  const int cluster = PAIR ? 2 : (p.cluster_k > 1 ? p.cluster_k : 1);
  using L = GemmSmem<BNC, STAGES>;
  auto kfn = gemm_kernel<BNC, STAGES, PAIR, F8>;
  constexpr int SMEM = (PAIR && BNC == 256) ? L::TOTAL_WIDE : L::TOTAL;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return TB200_ERR_CUDA;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_err(cudaLaunchKernelEx(&cfg, kfn, p));
}

template <bool F8>
static int launch_gemm(const GemmParams& p, const struct GemmPlan& plan, int sms, cudaStream_t stream);

static int set_operand(OperandGeom* g, CUtensorMap* tm, const void* base, long long rows_mn, long long k, long long ld,
                       int k_major, int eb, int tile_mn, CUtensorMapDataType dt) {
  if (k_major) {
    // memory: [rows_mn][k], K contiguous. One box = tile_mn rows x 128 bytes of K.
    const uint64_t dims[2] = {(uint64_t)k, (uint64_t)rows_mn};
    const uint64_t strides[1] = {(uint64_t)ld * eb};
    const uint32_t box[2] = {(uint32_t)(STAGE_K_BYTES / eb), (uint32_t)tile_mn};
    g->boxes = 1;
    g->box_bytes = tile_mn * STAGE_K_BYTES;
    g->box_mn = tile_mn;
    g->lbo = 16;
    g->sbo = 8 * STAGE_K_BYTES;
    g->kstep = 32;
    g->mn_major = 0;
    return encode_tmap(tm, dt, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  // memory: [k][rows_mn], MN contiguous (16-bit types only). One box = 64 MN elements x 64 k rows.
  if (eb != 2) return TB200_ERR_UNSUPPORTED;
  const uint64_t dims[2] = {(uint64_t)rows_mn, (uint64_t)k};
  const uint64_t strides[1] = {(uint64_t)ld * eb};
  const uint32_t box[2] = {64, 64};
  g->boxes = tile_mn / 64;
  g->box_bytes = 64 * 128;
  g->box_mn = 64;
  g->lbo = g->box_bytes;  // between 64-element MN groups
  g->sbo = 1024;          // between groups of 8 k rows
  g->kstep = 16 * 128;    // 16 k rows per MMA
  g->mn_major = 1;
  return encode_tmap(tm, dt, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int validate(const tb200_gemm_args* a) {
  if (!a || !a->a || !a->b || !a->c) return TB200_ERR_BAD_ARG;
  if (a->m < 0 || a->n < 0 || a->k < 0) return TB200_ERR_BAD_ARG;
  if (a->m > INT32_MAX || a->n > INT32_MAX || a->k > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  const int eb = elem_bytes(a->in_dtype);
  if (eb == 0) return TB200_ERR_UNSUPPORTED;
  if (a->out_dtype != TB200_BF16 && a->out_dtype != TB200_F16 && a->out_dtype != TB200_F32)
    return TB200_ERR_UNSUPPORTED;
  if (eb == 1 && (!a->a_k_major || !a->b_k_major)) return TB200_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15)) return TB200_ERR_BAD_ARG;
  if (((a->lda * eb) & 15) || ((a->ldb * eb) & 15)) return TB200_ERR_BAD_ARG;
  if (a->lda < (a->a_k_major ? a->k : a->m) || a->ldb < (a->b_k_major ? a->k : a->n) || a->ldc < a->n)
    return TB200_ERR_BAD_ARG;
  return TB200_OK;
}

template <bool F8>
static int launch_gemm(const GemmParams& p, const GemmPlan& plan, int sms, cudaStream_t stream) {
  if (plan.pair) {
    const int clusters = p.units < sms / 2 ? p.units : sms / 2;
    if (plan.pair == 2) return launch_one<256, 4, true, F8>(p, 2 * clusters, stream);
    return launch_one<128, 7, true, F8>(p, 2 * clusters, stream);
  }
  const int grid = p.units < sms ? p.units : sms;
  switch (plan.bn) {
    case 256: return launch_one<256, 4, false, F8>(p, grid, stream);
    case 128: return launch_one<128, 7, false, F8>(p, grid, stream);
    default: return launch_one<64, 8, false, F8>(p, grid, stream);
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* a) {
  if (validate(a) != TB200_OK) return 0;
  GemmPlan plan;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  if (!plan_gemm(a, sms, &plan)) return 0;
  if (plan.split_k <= 1 || plan.cluster_reduce) return 0;
  return (size_t)plan.split_k * (size_t)a->m * (size_t)a->n * sizeof(float);
}

extern "C" int tb200_gemm_plan(const tb200_gemm_args* a, int32_t* out6) {
  if (!out6) return TB200_ERR_BAD_ARG;
  int rc = validate(a);
  if (rc != TB200_OK) return rc;
  GemmPlan plan;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  if (!plan_gemm(a, sms, &plan)) return TB200_ERR_UNSUPPORTED;
  out6[0] = plan.pair ? 256 : BM;                       // rows of C per tile (per CTA pair when num_ctas = 2)
  out6[1] = plan.bn;                                    // columns of C per tile
  out6[2] = plan.pair ? 2 : 1;                          // CTAs that share a tile
  out6[3] = plan.split_k;
  out6[4] = plan.pair == 2 ? 4 : plan.pair == 1 ? 7 : plan.bn == 256 ? 4 : plan.bn == 128 ? 6 : 8;  // ring depth
  out6[5] = STAGE_K_BYTES / elem_bytes(a->in_dtype);    // K elements per ring stage
  return TB200_OK;
}

extern "C" int tb200_gemm(const tb200_gemm_args* a, void* stream_) {
  int rc = validate(a);
  if (rc != TB200_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->m == 0 || a->n == 0) return TB200_OK;
  const int out_eb = a->out_dtype == TB200_F32 ? 4 : 2;
  if (a->k == 0) {
    return cuda_err(cudaMemset2DAsync(a->c, (size_t)a->ldc * out_eb, 0, (size_t)a->n * out_eb, (size_t)a->m, stream));
  }
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;
  GemmPlan plan;
  if (!plan_gemm(a, sms, &plan)) return TB200_ERR_UNSUPPORTED;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int eb = elem_bytes(a->in_dtype);
  const bool f8 = eb == 1;
  CUtensorMapDataType dt = f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                              : (a->in_dtype == TB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  rc = set_operand(&p.ga, &p.tma, a->a, a->m, a->k, a->lda, a->a_k_major, eb, BM, dt);
  if (rc != TB200_OK) return rc;
  rc = set_operand(&p.gb, &p.tmb, a->b, a->n, a->k, a->ldb, a->b_k_major, eb, plan.pair == 2 ? 256 : plan.pair ? 128 : plan.bn, dt);
  if (rc != TB200_OK) return rc;

  uint32_t fmt;
  if (f8)
    fmt = a->in_dtype == TB200_E4M3 ? 0u : 1u;
  else
    fmt = a->in_dtype == TB200_F16 ? 0u : 1u;
  p.idesc = make_idesc(fmt, fmt, p.ga.mn_major, p.gb.mn_major, plan.pair ? 256 : BM, plan.pair ? 256 : plan.bn);
  p.c = a->c;
  p.ldc = a->ldc;
  p.m = (int)a->m;
  p.n = (int)a->n;
  p.k = (int)a->k;
  p.tiles_m = plan.tiles_m;
  p.tiles_n = plan.tiles_n;
  p.split_k = plan.split_k;
  p.kb_per_split = plan.kb_per_split;
  p.k_blocks = plan.k_blocks;
  p.units = plan.tiles_m * plan.tiles_n * plan.split_k;
  p.bk_elems = STAGE_K_BYTES / eb;
  p.group_m = 8;
  p.scale_a = a->scale_a;
  p.scale_b = a->scale_b;
  p.scale_mode = a->scale_mode;
  if (a->scale_mode == 1 && (!a->scale_a || !a->scale_b)) return TB200_ERR_BAD_ARG;
  if (a->scale_mode != 0 && a->scale_mode != 1) return TB200_ERR_UNSUPPORTED;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  const int final_mode = a->out_dtype == TB200_BF16 ? 0 : (a->out_dtype == TB200_F16 ? 1 : 2);
  if (plan.split_k > 1 && plan.cluster_reduce) {
    p.out_mode = final_mode;
    p.cluster_k = plan.split_k;
  } else if (plan.split_k > 1) {
    const size_t need = (size_t)plan.split_k * (size_t)a->m * (size_t)a->n * sizeof(float);
    if (!a->workspace || a->workspace_bytes < need) return TB200_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return TB200_ERR_BAD_ARG;
    p.ws = static_cast<float*>(a->workspace);
    p.out_mode = 3;
  } else {
    p.out_mode = final_mode;
  }
  if (plan.pair == 2 && p.out_mode <= 1 && (reinterpret_cast<uintptr_t>(a->c) & 15) == 0 && ((a->ldc * 2) & 15) == 0) {
    // wide tile, 16-bit output: the epilogue stores 64-column x 32-row boxes by TMA
    const uint64_t dims[2] = {(uint64_t)a->n, (uint64_t)a->m};
    const uint64_t strides[1] = {(uint64_t)a->ldc * 2};
    const uint32_t box[2] = {64, 32};
    rc = encode_tmap(&p.tmc, a->out_dtype == TB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     2, a->c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    p.c_tma = 1;
  }
  rc = f8 ? launch_gemm<true>(p, plan, sms, stream) : launch_gemm<false>(p, plan, sms, stream);
  if (rc != TB200_OK) return rc;
  if (plan.split_k > 1 && !plan.cluster_reduce) {
    // scale factors were already applied to the partial sums
    const long long total = (long long)a->m * ((a->n + 3) / 4);
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    rc = cuda_err(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, (const float*)p.ws, a->c, p.m, p.n, p.ldc, plan.split_k,
                                     final_mode));
  }
  return rc;
}
