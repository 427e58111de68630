// Grouped (per-expert) GEMM for MoE layers on sm_100a with the routing gather fused into the TMA
// load and the scatter / gate scaling / SwiGLU fused into the epilogue:
//
//   for each expert e and each sorted row r in [slice_offs[e], slice_offs[e+1]):
//       acc      = X[gather[r], :] @ W[e]            (+ bias[e])
//       acc      = swiglu(acc)                        (optional; interleaved gate / linear columns)
//       Y[scatter[r], :] = acc * gammas[r]            (scatter[r] == -1: dropped)
//
// Work units are (block-schedule entry, N tile): the schedule lists the 128-row blocks of every
// non-empty expert as (block << 16) | expert, padded with -1, so a tile never straddles experts.
// A tile, no gather (rows already expert-sorted): one tiled TMA box per K step.
// A tile, gathered: four gather warps copy the 128 indexed rows with 16-byte asynchronous copies
// (LDGSTS) directly into the swizzled shared-memory layout, two K steps in flight, and signal the
// stage's barrier after a proxy fence. (`cp.async.bulk.tensor.2d.tile::gather4`, which the
// reference uses, was measured first: 32 four-row copies per K step ran the 65536 x 4096 x 3072
// GEMM at 400 TFLOP/s against 980 with tiled loads, so the row gather moved to LDGSTS.)
// W[e] is read through a 3-D tensor map (expert is the outermost coordinate), K-major or N-major.
// MMA issue, TMEM double buffering and the lean single-thread loops are those of the dense kernel.
//
// Counterpart in the reference: _p_matmul, python/triton_kernels/triton_kernels/matmul_details/
// _p_matmul.py:62-790 (gather :343-344, bias/activation/gammas :561-622, scatter :733-737), host
// entry triton_kernels/matmul.py:243.
#include <string.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "host_common.h"
#include "moe_epilogue.cuh"

namespace tb200 {

static constexpr int MOE_THREADS = 320;  // TMA warp, MMA warp, 4 epilogue warps, 4 gather warps
static constexpr int MOE_BM = 128;
static constexpr int MOE_BN = 256;

struct MoeParams {
  CUtensorMap tmx_tile;  // X: (K, rows_x), box (64, 128): contiguous-row source (no gather)
  CUtensorMap tmw;  // W: K-major (K, N, E) box (64, BN, 1); N-major (N, K, E) box (64, 64, 1)
  const int* slice_offs;
  const int* slice_sizes;  // optional: rows of expert e = slice_sizes[e] (else slice_offs[e+1] - slice_offs[e])
  const int* sched;
  const int* gather;
  const int* scatter;
  const float* gammas;
  const float* bias;
  const uint16_t* x;  // gather source (16-bit elements)
  long long ldx;
  void* y;
  int* status;
  long long ldy;
  int n_sched, tiles_n, units;
  int n, k, k_blocks, rows_x, rows_y;
  int w_n_major;
  int swiglu, has_limit, out_f16;
  float alpha, limit;
  uint32_t idesc;
  // fused combine: when y_world > 0 the row with output index i is stored to row i % rows_per_peer of
  // y_peers[i / rows_per_peer] (buffers of other GPUs, mapped by CUDA IPC; plain st.global)
  int y_world;
  int rows_per_peer;
  int gammas_by_out_row;
  void* y_peers[16];
  const float* betas;    // optional per sorted row factor on the bias
  float out_alpha;       // factor on the biased accumulator (1 when unused)
  const void* acc_in;    // optional 16-bit matrix added to the result (rows as in y, no scatter)
  long long ld_acc;
  // MX-quantised output: y holds fp8 bytes (ldy in bytes), y_sf one e8m0 scale per 32 outputs of a row
  uint8_t* y_sf;
  long long ld_ysf;
  int mx_kind;  // MOE_OUT_E4M3 / MOE_OUT_E5M2
};

// 16-byte asynchronous copy global -> shared (LDGSTS); src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_load_3d_a(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int x, int y, int z,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y, int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}

// BNC = W rows (N) staged per CTA. Single: 128 x 256 tile per CTA, 4 stages. Pair: a 2-CTA cluster
// shares a 256-row x 256-column tile (two consecutive 128-row blocks of one expert; schedule entries
// with an odd block index are covered by their even neighbour), CTA r stages rows block+r of A
// and W rows [n0 + 128 r, +128), the leader issues tcgen05.mma.cta_group::2: 32 KB per K step per
// CTA instead of 48 KB and a 6-deep ring.
template <bool PAIR>
struct MoeCfg {
  static constexpr int BNC = PAIR ? 128 : 256;
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int A_BYTES = MOE_BM * 128;
  static constexpr int B_BYTES = BNC * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // one 4 KB staging buffer (32 rows x 128 bytes) per epilogue warp, 256 bytes past the barriers: rows that leave the
  // GPU are transposed through it so that a store instruction writes whole 128-byte lines of four rows
  static constexpr int EPI_OFFSET = BAR_OFFSET + 256;
  // pair mode: the schedule entries a cluster works on (even blocks), compacted once per CTA so that the static
  // round-robin over units gives every cluster the same number of tiles (skipping the odd entries in place left
  // the clusters with binomially spread loads: 53 +- 5 tiles each, the slowest one a quarter above the mean). The
  // list holds what a cluster works on (at most ACT_CAP entries, else the kernel falls back to skipping in place);
  // the schedule it is cut from may be ten times longer, being sized for the worst case and padded with -1.
  static constexpr int ACT_CAP = PAIR ? 4096 : 0;
  static constexpr int ACT_OFFSET = EPI_OFFSET + 4 * 4096;
  static constexpr int TOTAL = ACT_OFFSET + (PAIR ? ACT_CAP * 4 + 64 : 0) + 1024;
  // K steps a gather warp keeps in flight. At most stages - 2: the MMA thread releases stage i only after the
  // first MMA of step i + 1, which needs step i + 1 signalled - with stages - 1 steps held back the gather
  // would wait for a stage whose release waits for the gather (measured: a 2 s bounded-wait timeout).
  static constexpr int LOOKAHEAD = PAIR ? 3 : 2;
};

// MXOUT: the instantiation whose epilogue can MX-quantise the output; the plain one compiles that branch out (it
// cost the plain kernel spills at its 168-register cap).
template <bool PAIR, bool MXOUT>
__global__ void __launch_bounds__(MOE_THREADS, 1) moe_gemm_kernel(const __grid_constant__ MoeParams p) {
  using L = MoeCfg<PAIR>;
  constexpr int BN = MOE_BN;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const bool gathered = p.gather != nullptr;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmx_tile);
    tma_prefetch_desc(&p.tmw);
    for (int s = 0; s < STAGES; ++s) {
      // the expect_tx arrival, plus one arrival per gather warp (of both CTAs in pair mode)
      mbar_init(&full[s], gathered ? (PAIR ? 9 : 5) : 1);
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

  int units = p.units;
  const int tiles_n = p.tiles_n, k_blocks = p.k_blocks;
  const int* sched = p.sched;
  bool compact = false;
  if constexpr (PAIR) {
    {
      // two passes over the schedule by all warps: count the active entries of a warp's chunk, then write them
      // (the schedule may be much longer than the list: it is sized for the worst case and padded with -1)
      int* const act = reinterpret_cast<int*>(smem + L::ACT_OFFSET);
      int* const cnt = act + L::ACT_CAP;
      constexpr int NW = MOE_THREADS / 32;
      const int chunk = ((p.n_sched + NW - 1) / NW + 31) & ~31;
      const int lo = warp * chunk, hi = min(p.n_sched, lo + chunk);
      int mine = 0;
      for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        const int en = i < hi ? __ldg(p.sched + i) : -1;
        mine += __popc(__ballot_sync(0xffffffffu, en >= 0 && ((en >> 16) & 1) == 0));
      }
      if (lane == 0) cnt[warp] = mine;
      __syncthreads();
      int pos = 0, total = 0;
      for (int w = 0; w < NW; ++w) {
        const int c = cnt[w];
        if (w < warp) pos += c;
        total += c;
      }
      if (total <= L::ACT_CAP) {  // the same for every thread of the CTA
        for (int base = lo; base < hi; base += 32) {
          const int i = base + lane;
          const int en = i < hi ? __ldg(p.sched + i) : -1;
          const bool on = en >= 0 && ((en >> 16) & 1) == 0;
          const uint32_t m = __ballot_sync(0xffffffffu, on);
          if (on) act[pos + __popc(m & ((1u << lane) - 1u))] = en;
          pos += __popc(m);
        }
        __syncthreads();
        sched = act;
        units = total * tiles_n;
        compact = true;
      }
    }
  }
  const int* const slice_offs = p.slice_offs;
  const int* const slice_sizes = p.slice_sizes;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);
  const uint32_t leader_full = PAIR ? mapa_shared(full_a, 0) : full_a;

  // A schedule entry is worked on iff it is valid and (pair mode) names an even block.
  auto entry_active = [&](int entry) -> bool { return entry >= 0 && (!PAIR || (((entry >> 16) & 1) == 0)); };
  // schedule entry si: from the compacted list in shared memory (pair mode) or from global memory
  auto sched_at = [&](int si) -> int { return compact ? sched[si] : __ldg(sched + si); };

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (one lane)
    if (lane == 0) {
      // measured at 65536 rows x 128 experts against the other combinations of evict_first / normal / last: this
      // one is the fastest or within 1 % of it for both GEMMs of the layer. (TMA prefetches into L2 of the boxes 8 to
      // 24 K steps ahead of the loads, the next tile's first steps included, made the layer's GEMMs 30 % slower.)
      const uint64_t pol_x = policy_evict_normal();
      const uint64_t pol_w = policy_evict_last();
      const int w_n_major = p.w_n_major;
      const uint32_t tx_bytes = (gathered ? L::B_BYTES : L::STAGE_BYTES) * (PAIR ? 2 : 1);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = worker; unit < units && ok; unit += num_workers) {
        const int si = unit / tiles_n;
        const int entry = sched_at(si);
        if (!entry_active(entry)) continue;
        const int e = entry & 0xFFFF;
        const int n0 = (unit - si * tiles_n) * BN + (int)rank * L::BNC * (PAIR ? 1 : 0);
        const int row0 = __ldg(slice_offs + e) + ((entry >> 16) + (int)rank) * MOE_BM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx_a(full_a + s * 8, tx_bytes);
          const uint32_t bar = leader_full + s * 8;
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          const int kx = kb * 64;
          // Without a gather the sorted rows are contiguous: one tiled box (rows past the slice end
          // belong to the next expert; their products are never stored).
          if (!gathered) {
            if constexpr (PAIR) tma_load_2d_pair(sa, &p.tmx_tile, bar, kx, row0, pol_x);
            else tma_load_2d_a(sa, &p.tmx_tile, bar, kx, row0, pol_x);
          }
          const uint32_t sb = sa + L::A_BYTES;
          if (w_n_major) {
#pragma unroll
            for (int i = 0; i < L::BNC / 64; ++i) {
              if constexpr (PAIR) tma_load_3d_pair(sb + i * 8192, &p.tmw, bar, n0 + i * 64, kx, e, pol_w);
              else tma_load_3d_a(sb + i * 8192, &p.tmw, bar, n0 + i * 64, kx, e, pol_w);
            }
          } else {
            if constexpr (PAIR) tma_load_3d_pair(sb, &p.tmw, bar, kx, n0, e, pol_w);
            else tma_load_3d_a(sb, &p.tmw, bar, kx, n0, e, pol_w);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------- gather warps (A rows by index)
    // 128 threads copy the 128 x 128-byte A tile of each K step with 16-byte LDGSTS copies straight
    // into the 128-byte-swizzled layout the MMA descriptor expects (chunk c of row r lands at
    // r * 128 + ((c ^ (r & 7)) << 4)); rows past the expert's slice are zero-filled. Each thread
    // keeps LOOKAHEAD K steps in flight; when a step has landed it fences the writes for the async
    // proxy and its warp arrives on the stage's `full` barrier (the leader's, in pair mode).
    if (gathered) {
      const int gt = threadIdx.x - 192;
      const int chunk = gt & 7, rsub = gt >> 3;
      const int* const gather = p.gather;
      const uint16_t* const x = p.x;
      const long long ldx = p.ldx;
      const int rows_x = p.rows_x, kdim = p.k;
      uint32_t s = 0, ph = 0;      // stage being filled
      uint32_t s_old = 0;          // oldest stage issued but not yet signalled
      uint32_t pending = 0;        // K steps issued but not yet signalled
      bool ok = true;
      auto signal_oldest = [&]() {
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(leader_full + s_old * 8);
          else mbar_arrive_a(full_a + s_old * 8);
        }
        if (++s_old == STAGES) s_old = 0;
        --pending;
      };
      for (int unit = worker; unit < units && ok; unit += num_workers) {
        const int si = unit / tiles_n;
        const int entry = sched_at(si);
        if (!entry_active(entry)) continue;
        const int e = entry & 0xFFFF;
        const int row0 = __ldg(slice_offs + e) + ((entry >> 16) + (int)rank) * MOE_BM;
        const int row_end = slice_sizes ? __ldg(slice_offs + e) + __ldg(slice_sizes + e) : __ldg(slice_offs + e + 1);
        const uint16_t* src[8];
        uint32_t dst_off[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rsub + 16 * i;
          const int sr = row0 + r;
          int row = -1;
          if (sr < row_end) {
            row = __ldg(gather + sr);
            if (row >= rows_x) row = -1;
          }
          src[i] = row >= 0 ? x + (long long)row * ldx + chunk * 8 : nullptr;
          dst_off[i] = (uint32_t)(r * 128 + ((chunk ^ (r & 7)) << 4));
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          const int kx = kb * 64;
          const bool k_in = kx + chunk * 8 < kdim;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool v = k_in && src[i] != nullptr;
            cp_async_16(sa + dst_off[i], v ? (const void*)(src[i] + kx) : (const void*)x, v ? 16u : 0u);
          }
          cp_async_commit();
          ++pending;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
          if (pending > L::LOOKAHEAD) {
            cp_async_wait<L::LOOKAHEAD>();
            fence_proxy_async_smem();
            __syncwarp();
            signal_oldest();
          }
        }
      }
      // drain
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      while (pending > 0) signal_oldest();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = p.idesc;
      const uint32_t b_lbo = p.w_n_major ? 8192u : 16u;
      const uint64_t bk = p.w_n_major ? (uint64_t)(2048 >> 4) : (uint64_t)(32 >> 4);
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, b_lbo, 1024, SWIZZLE_128B);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      const uint32_t peer_delta = PAIR ? (mapa_shared(empty_a, 1) - empty_a) : 0u;
      uint32_t s = 0, ph = 0, tcount = 0;
      bool ok = true;
      auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t acc) {
        if constexpr (PAIR) umma_f16_ss_pair(d, a, b, idesc, acc);
        else umma_f16_ss(d, a, b, idesc, acc);
      };
      auto commit = [&](uint32_t bar) {
        if constexpr (PAIR) {
          umma_commit_pair(bar);
          umma_commit_pair(bar + peer_delta);
        } else {
          umma_commit_a(bar);
        }
      };
      for (int unit = worker; unit < units && ok; unit += num_workers) {
        const int si = unit / tiles_n;
        if (!entry_active(sched_at(si))) continue;
        const uint32_t acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait_a(tempty_a + acc * 8, aph ^ 1, status, WAIT_TMEM_EMPTY)) break;
        if (!mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        uint32_t accum = 0;
        uint32_t prev_empty = 0;
        for (int i = 0; i < k_blocks; ++i) {
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          mma(tmem_d, ad, bd, accum);
          accum = 1u;
          if (prev_empty) commit(prev_empty);
          prev_empty = empty_a + s * 8;
          mma(tmem_d, ad + 2, bd + bk, 1u);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
          if (i + 1 < k_blocks) {
            if (!mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          mma(tmem_d, ad + 4, bd + 2 * bk, 1u);
          mma(tmem_d, ad + 6, bd + 3 * bk, 1u);
        }
        if (ok) {
          commit(prev_empty);
          commit(tfull_a + acc * 8);
        }
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const int* const scatter = p.scatter;
    const float* const gammas = p.gammas;
    const float* const bias = p.bias;
    const int n = p.n, swiglu = p.swiglu, has_limit = p.has_limit, out_f16 = p.out_f16, rows_y = p.rows_y;
    const float alpha = p.alpha, limit = p.limit;
    const long long ldy = p.ldy;
    uint16_t* const y_local = reinterpret_cast<uint16_t*>(p.y);
    const int y_world = p.y_world, rows_per_peer = p.rows_per_peer, gammas_by_out_row = p.gammas_by_out_row;
    const uint32_t tempty_leader = PAIR ? mapa_shared(smem_u32(tempty), 0) : smem_u32(tempty);
    uint32_t tcount = 0;
    for (int unit = worker; unit < units; unit += num_workers) {
      const int si = unit / tiles_n;
      const int entry = sched_at(si);
      if (!entry_active(entry)) continue;
      const int e = entry & 0xFFFF;
      const int n0 = (unit - si * tiles_n) * BN;
      const int row0 = __ldg(slice_offs + e) + ((entry >> 16) + (int)rank) * MOE_BM;
      const int row_end = slice_sizes ? __ldg(slice_offs + e) + __ldg(slice_sizes + e) : __ldg(slice_offs + e + 1);
      const uint32_t acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&tfull[acc], aph, status, WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int sr = row0 + q * 32 + lane;  // sorted row handled by this thread
      int out_row = -1;
      float gamma = 1.f;
      uint16_t* y = y_local;
      MoeEpilogueExtra extra;
      extra.out_alpha = p.out_alpha;
      extra.acc_in = p.acc_in;
      extra.ld_acc = p.ld_acc;
      if (sr < row_end) {
        out_row = scatter ? __ldg(scatter + sr) : sr;
        if (out_row >= rows_y) out_row = -1;
        if (gammas) gamma = gammas_by_out_row ? (out_row >= 0 ? __ldg(gammas + out_row) : 0.f) : __ldg(gammas + sr);
        if (y_world > 0 && out_row >= 0) {
          const int to = out_row / rows_per_peer;
          y = static_cast<uint16_t*>(p.y_peers[to]);
          out_row -= to * rows_per_peer;
        }
        if (p.betas) extra.beta = __ldg(p.betas + sr);
      }
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      const float* brow = bias ? bias + (long long)e * n : nullptr;
      if (y_world > 0 && !swiglu && !p.acc_in && (ldy & 7) == 0) {
        // Fused combine: this warp's 32 rows go to other GPUs' buffers. A thread owns a row, so storing its 64 columns
        // directly puts 32 rows x 32 bytes into every instruction - 32-byte packets over NVLink, measured at a quarter
        // of the link rate (GEMM-2 of the expert-parallel layer: 0.56 ms at 4 GPUs against 0.24 for the same tiles
        // stored locally). Instead the 64 columns (128 bytes) of all 32 rows are written to a swizzled staging buffer
        // and read back transposed: eight lanes cover one row's 128-byte line, an instruction writes four whole lines.
        const uint32_t stage = smem_a + L::EPI_OFFSET + (uint32_t)q * 4096;
        uint8_t* const row_ptr = out_row >= 0 ? reinterpret_cast<uint8_t*>(y) + (long long)out_row * ldy * 2 : nullptr;
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 64) {
          const int col = n0 + cc;
          if (col >= n) break;
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(taddr + cc, v0);
          tmem_ld_32x32b_x32(taddr + cc + 32, v1);
          tmem_ld_wait();
          if (col + 64 > n) {  // ragged last columns: per-thread stores
            if (out_row >= 0) {
              moe_store_chunk(v0, y, ldy, out_row, col, n, brow, swiglu, alpha, limit, has_limit, gamma, out_f16, 1.f, extra);
              if (col + 32 < n)
                moe_store_chunk(v1, y, ldy, out_row, col + 32, n, brow, swiglu, alpha, limit, has_limit, gamma, out_f16, 1.f, extra);
            }
            continue;
          }
          uint32_t w[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float a0 = __uint_as_float(v0[2 * j]), a1 = __uint_as_float(v0[2 * j + 1]);
            float b0 = __uint_as_float(v1[2 * j]), b1 = __uint_as_float(v1[2 * j + 1]);
            if (brow) {
              a0 += __ldg(brow + col + 2 * j) * extra.beta;
              a1 += __ldg(brow + col + 2 * j + 1) * extra.beta;
              b0 += __ldg(brow + col + 32 + 2 * j) * extra.beta;
              b1 += __ldg(brow + col + 33 + 2 * j) * extra.beta;
            }
            const float sc = extra.out_alpha * gamma;
            w[j] = moe_pack16(a0 * sc, a1 * sc, out_f16);
            w[16 + j] = moe_pack16(b0 * sc, b1 * sc, out_f16);
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t addr = stage + (uint32_t)lane * 128 + ((uint32_t)(c ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                         "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                         : "memory");
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3), c = lane & 7;
            uint4 val;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                         : "r"(stage + (uint32_t)r * 128 + ((uint32_t)(c ^ (r & 7)) << 4))
                         : "memory");
            uint8_t* dst = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, (unsigned long long)row_ptr, r));
            if (dst) *reinterpret_cast<uint4*>(dst + (long long)col * 2 + c * 16) = val;
          }
          __syncwarp();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(tempty_leader + acc * 8);
          else mbar_arrive_a(tempty_leader + acc * 8);
        }
        continue;
      }
      if (MXOUT && p.y_sf) {
        // MX-quantised output: a block of 32 outputs is one chunk of 32 accumulator columns, or two with SwiGLU
        const int step = swiglu ? 64 : 32;
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += step) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(taddr + cc, v0);
          if (swiglu) tmem_ld_32x32b_x32(taddr + cc + 32, v1);
          tmem_ld_wait();
          const int col = n0 + cc;
          if (out_row < 0 || col >= n) continue;
          float o[32];
          moe_chunk_values<0>(v0, col, n, brow, swiglu, alpha, limit, has_limit, gamma, 1.f, extra, o);
          int ocol = col, cnt = min(32, n - col);
          if (swiglu) {
            moe_chunk_values<16>(v1, col + 32, n, brow, 1, alpha, limit, has_limit, gamma, 1.f, extra, o);
            ocol = col >> 1;
            cnt = min(32, (n - col) >> 1);
          }
          moe_store_mx_block(o, cnt, y, (long long)out_row * ldy + ocol, p.y_sf + (long long)out_row * p.ld_ysf + (ocol >> 5),
                             p.mx_kind);
        }
      } else {
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + cc, v);
          tmem_ld_wait();
          const int col = n0 + cc;
          if (out_row < 0 || col >= n) continue;
          moe_store_chunk(v, y, ldy, out_row, col, n, brow, swiglu, alpha, limit, has_limit, gamma, out_f16, 1.f, extra);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(tempty_leader + acc * 8);
        else mbar_arrive_a(tempty_leader + acc * 8);
      }
    }
  }

  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool PAIR>
static int launch_moe(const MoeParams& p, int sms, cudaStream_t stream) {
  using L = MoeCfg<PAIR>;
  auto kfn = p.y_sf ? moe_gemm_kernel<PAIR, true> : moe_gemm_kernel<PAIR, false>;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  const int workers_max = PAIR ? sms / 2 : sms;
  const int workers = p.units < workers_max ? p.units : workers_max;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(PAIR ? 2 * workers : workers);
  cfg.blockDim = dim3(MOE_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_err(cudaLaunchKernelEx(&cfg, kfn, p));
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_moe_gemm(const tb200_moe_gemm_args* a, void* stream_) {
  if (!a || !a->x || !a->w || !a->slice_offs || !a->block_schedule) return TB200_ERR_BAD_ARG;
  if (a->y_world < 0 || a->y_world > 16) return TB200_ERR_BAD_ARG;
  if (a->c_acc_in && (a->scatter_indx || a->y_world > 0 || a->ld_acc_in <= 0)) return TB200_ERR_UNSUPPORTED;
  if (a->y_mx_scale) {
    if (a->c_acc_in || a->y_world > 0) return TB200_ERR_UNSUPPORTED;
    if (a->y_mx_dtype != TB200_E4M3 && a->y_mx_dtype != TB200_E5M2) return TB200_ERR_BAD_ARG;
    if (a->ld_y_mx_scale < ((a->swiglu ? a->n / 2 : a->n) + 31) / 32) return TB200_ERR_BAD_ARG;
  }
  if (a->y_world == 0 && !a->y) return TB200_ERR_BAD_ARG;
  if (a->y_world > 0) {
    if (!a->y_peers || a->rows_per_peer <= 0 || a->rows_per_peer > INT32_MAX) return TB200_ERR_BAD_ARG;
    for (int i = 0; i < a->y_world; ++i)
      if (!a->y_peers[i] || (reinterpret_cast<uintptr_t>(a->y_peers[i]) & 15)) return TB200_ERR_BAD_ARG;
    if (a->rows_y > (int64_t)a->y_world * a->rows_per_peer) return TB200_ERR_BAD_ARG;
  }
  if (a->n_experts <= 0 || a->n_experts > 65535 || a->k <= 0 || a->n <= 0 || a->n_sched < 0) return TB200_ERR_BAD_ARG;
  if (a->rows_x < 0 || a->rows_y < 0) return TB200_ERR_BAD_ARG;
  if (a->dtype != TB200_BF16 && a->dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (a->swiglu && (a->n & 1)) return TB200_ERR_BAD_ARG;
  if ((a->k % 8) || (a->ldx % 8) || (a->w_n_major && (a->n % 8))) return TB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & 15)) return TB200_ERR_BAD_ARG;
  if (a->rows_x > INT32_MAX - 1 || a->rows_y > INT32_MAX || a->k > INT32_MAX || a->n > INT32_MAX)
    return TB200_ERR_UNSUPPORTED;
  if (a->n_sched == 0 || a->rows_x == 0) return TB200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  // Tilings. One CTA per 128-row block (128 x 256 tile), or a CTA pair per two consecutive blocks of an expert
  // (256 x 256, moe_tile_mode 2): the pair stages a third less per K step (GEMM-1 with 512-row experts: 1100-1215
  // TFLOP/s against 920-1000) but pads routed expert sizes to 256 rows (25 % instead of 12 %), and loses 2x on
  // gathered rows (eight remote barrier arrivals per K step from the peer's gather warps). A third tiling, 256 rows x
  // 512 columns per pair with one 512-column accumulator (the dense kernel's wide tile), ran GEMM-1 at 590-800
  // TFLOP/s against 930: its epilogue (SwiGLU, scattered per-thread stores) cannot hide behind a second accumulator.
  // A mix (pairs for the blocks that have a partner, then a second launch with one CTA per leftover block, so that
  // no pair carries a padded half) measured 3-8 % behind the pure pair tiling: the leftover blocks re-read their
  // experts' weights from HBM (1.65 GB at 128 experts) instead of sharing them in L2 with the expert's other tiles.
  // The epilogue is not what bounds either tiling: with the four gather warps (idle when the rows are sorted) as a
  // second epilogue group, each group converting and storing half of a tile's columns, the 16384-token layer
  // measured 2.89-2.90 ms against 2.85-2.88.
  // The choice: the pair tiling for sorted (not gathered) rows when the experts average at least 256 rows. Both
  // GEMMs of a layer, routed expert sizes, pair against one CTA per block: 8192 / 16384 / 32768 / 49152 rows on
  // 16 / 32 / 64 / 96 experts 0.354 / 0.695 / 1.29 / 2.01 ms against 0.375 / 0.725 / 1.40 / 2.28 ms; 65536 rows on
  // 128 experts 2.87 against 3.11 ms (alternating in one process, six rounds, the pair ahead in each).
  const bool pair = a->moe_tile_mode == 2 ||
                    (a->moe_tile_mode == 0 && !a->gather_indx && sms >= 2 && a->rows_x >= 256 * a->n_experts);
  MoeParams p;
  memset(&p, 0, sizeof(p));
  const CUtensorMapDataType dt =
      a->dtype == TB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->rows_x};
    const uint64_t strides[1] = {(uint64_t)a->ldx * 2};
    const uint32_t box_tile[2] = {64, 128};
    int rc = encode_tmap(&p.tmx_tile, dt, 2, a->x, dims, strides, box_tile, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  if (a->w_n_major) {
    const uint64_t dims[3] = {(uint64_t)a->n, (uint64_t)a->k, (uint64_t)a->n_experts};
    const uint64_t strides[2] = {(uint64_t)a->n * 2, (uint64_t)a->n * a->k * 2};
    const uint32_t box[3] = {64, 64, 1};
    int rc = encode_tmap(&p.tmw, dt, 3, a->w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  } else {
    const uint64_t dims[3] = {(uint64_t)a->k, (uint64_t)a->n, (uint64_t)a->n_experts};
    const uint64_t strides[2] = {(uint64_t)a->k * 2, (uint64_t)a->n * a->k * 2};
    const uint32_t box[3] = {64, (uint32_t)(pair ? 128 : MOE_BN), 1};
    int rc = encode_tmap(&p.tmw, dt, 3, a->w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.slice_offs = a->slice_offs;
  p.slice_sizes = a->slice_sizes;
  p.sched = a->block_schedule;
  p.gather = a->gather_indx;
  p.scatter = a->scatter_indx;
  p.gammas = a->gammas;
  p.bias = a->bias;
  p.x = static_cast<const uint16_t*>(a->x);
  p.ldx = a->ldx;
  p.y = a->y;
  p.ldy = a->ldy;
  p.gammas_by_out_row = a->gammas_by_out_row ? 1 : 0;
  p.betas = a->betas;
  p.out_alpha = a->has_out_alpha ? a->out_alpha : 1.f;
  p.acc_in = a->c_acc_in;
  p.ld_acc = a->ld_acc_in;
  p.y_world = a->y_world;
  p.rows_per_peer = (int)a->rows_per_peer;
  for (int i = 0; i < a->y_world; ++i) p.y_peers[i] = a->y_peers[i];
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.y_sf = static_cast<uint8_t*>(a->y_mx_scale);
  p.ld_ysf = a->ld_y_mx_scale;
  p.mx_kind = a->y_mx_dtype == TB200_E5M2 ? MOE_OUT_E5M2 : MOE_OUT_E4M3;
  p.n_sched = a->n_sched;
  p.tiles_n = (int)((a->n + MOE_BN - 1) / MOE_BN);
  const long long units = (long long)a->n_sched * p.tiles_n;
  if (units > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  p.units = (int)units;
  p.n = (int)a->n;
  p.k = (int)a->k;
  p.k_blocks = (int)((a->k + 63) / 64);
  p.rows_x = (int)a->rows_x;
  p.rows_y = (int)a->rows_y;
  p.w_n_major = a->w_n_major ? 1 : 0;
  p.swiglu = a->swiglu ? 1 : 0;
  p.has_limit = a->swiglu_has_limit ? 1 : 0;
  p.alpha = a->swiglu_alpha;
  p.limit = a->swiglu_limit;
  p.out_f16 = a->dtype == TB200_F16 ? 1 : 0;
  const uint32_t fmt = a->dtype == TB200_F16 ? 0u : 1u;
  p.idesc = make_idesc(fmt, fmt, 0u, p.w_n_major ? 1u : 0u, pair ? 256 : MOE_BM, MOE_BN);
  return pair ? launch_moe<true>(p, sms, stream) : launch_moe<false>(p, sms, stream);
}
