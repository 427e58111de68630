// MXFP8 block-scaled GEMM for sm_100a: C[M,N] = (A * sA) (B * sB)^T with A [M,K] and B [N,K] in
// e4m3, one e8m0 scale per 1x32 block along K, fp32 accumulation in tensor memory, bf16 output.
//
// Same skeleton as the dense kernel (TMA producer warp, single-thread MMA issuer, four epilogue
// warps, persistent grouped tile order). Per K step (128 elements = 4 MMAs of K = 32):
//   * the producer lands A (128 x 128 B), B (BN x 128 B) with 128-byte-swizzled TMA boxes, plus
//     one 512-byte scale atom per 128 operand rows with an untiled bulk copy. The scale tensors
//     are stored in the 512-byte-atom order [row/128][K/128][row%32][row/32%4][k%4], so the atom
//     for (row block, K step) is one contiguous run.
//   * the MMA thread copies each atom to tensor memory with tcgen05.cp.32x128b.warpx4 (32 rows x
//     16 bytes, replicated to the four lane quarters: lane = row % 32, column = row / 32 % 4, byte
//     = k % 4) and issues tcgen05.mma.kind::mxf8f6f4.block_scale; the instruction descriptor's
//     scale-factor ids pick byte k of the scale columns for the k-th MMA of the step.
// Tensor memory: BN = 256 keeps one 256-column accumulator plus 32 scale columns (epilogue not
// overlapped with the next tile); BN = 128 double-buffers the accumulator.
//
// Counterpart in the reference: _gemm_mxfp8_ws_kernel,
// third_party/tlx/tutorials/blackwell_gemm_ws_mxfp8.py:751-1035 (producer :616-698, MMA :563-613,
// epilogue :511-560); scale layout python/triton_kernels/triton_kernels/tensor_details/
// layout_details/blackwell_scale.py:100-122.
#include <string.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int MX_BM = 128;
static constexpr int MX_THREADS = 192;

struct MxParams {
  CUtensorMap tma;
  CUtensorMap tmb;
  const uint8_t* sfa;  // swizzled e8m0 scales of A
  const uint8_t* sfb;  // swizzled e8m0 scales of B
  void* c;
  int* status;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n, units;
  int k_blocks;   // K / 128
  int n_blocks;   // N / 128
  int group_m;
};

template <int BN, int STAGES>
struct MxSmem {
  static constexpr int A_BYTES = MX_BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SF_BYTES = 512 + (BN / 128) * 512;  // per stage: SFA atom + SFB atoms
  static constexpr int SF_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = SF_OFFSET + STAGES * SF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(MX_THREADS, 1) gemm_mxfp8_kernel(const __grid_constant__ MxParams p) {
  using L = MxSmem<BN, STAGES>;
  constexpr int NACC = (BN == 256) ? 1 : 2;
  constexpr int NB = BN / 128;  // scale atoms of B per K step
  constexpr uint32_t SF_COL0 = NACC * BN;  // first scale column; two sets of 16 columns
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

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma);
    tma_prefetch_desc(&p.tmb);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
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

  const int units = p.units, group_m = p.group_m, tiles_m = p.tiles_m, tiles_n = p.tiles_n;
  const int k_blocks = p.k_blocks, n_blocks = p.n_blocks;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      const uint8_t* const sfa = p.sfa;
      const uint8_t* const sfb = p.sfb;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const TileCoord t = unit_to_tile(unit, 1, group_m, tiles_m, tiles_n);
        const int m0 = t.pid_m * MX_BM, n0 = t.pid_n * BN;
        const int nb_valid = min(NB, n_blocks - t.pid_n * NB);  // 128-row blocks of B inside N
        const uint8_t* a_atoms = sfa + (size_t)t.pid_m * k_blocks * 512;
        const uint8_t* b_atoms = sfb + (size_t)t.pid_n * NB * k_blocks * 512;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = full_a + s * 8;
          mbar_expect_tx_a(bar, L::STAGE_BYTES + 512 + nb_valid * 512);
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          tma_load_2d_a(sa, &p.tma, bar, kb * 128, m0, pol);
          tma_load_2d_a(sa + L::A_BYTES, &p.tmb, bar, kb * 128, n0, pol);
          uint8_t* sf = smem + L::SF_OFFSET + s * L::SF_BYTES;
          bulk_load(sf, a_atoms + (size_t)kb * 512, 512, &full[s]);
          for (int j = 0; j < nb_valid; ++j)
            bulk_load(sf + 512 + j * 512, b_atoms + ((size_t)j * k_blocks + kb) * 512, 512, &full[s]);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t idesc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) idesc[k] = make_idesc_mx(0u, 0u, MX_BM, BN, (uint32_t)k, (uint32_t)k);
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, 16, 1024, SWIZZLE_128B);
      // scale atoms: 32 rows x 16 bytes, rows contiguous (no swizzle): 8-row groups 128 bytes apart
      const uint64_t sfdesc0 = make_smem_desc(smem_a + L::SF_OFFSET, 16, 128, SWIZZLE_NONE);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      uint32_t s = 0, ph = 0, tcount = 0, kpar = 0;
      bool ok = true, ready = false;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
        const uint32_t acc = tcount % NACC;
        const uint32_t aph = (tcount / NACC) & 1;
        if (!mbar_wait_a(tempty_a + acc * 8, aph ^ 1, status, WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        // Simple order per K step: wait, scale copies, four MMAs, commit. (Deferring the commit and
        // waiting for the next stage between the MMAs, which gains 10 % in the dense kernel, lost
        // 5-10 % here, and scale copies placed between MMAs lost 13 %.)
        uint32_t accum = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready && !mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          {  // probe the next stage ahead of this stage's MMAs (a blocking wait costs ~70 cycles even when ready)
            const uint32_t s1 = (s + 1 == STAGES) ? 0 : s + 1;
            ready = mbar_test_a(full_a + s1 * 8, s1 == 0 ? ph ^ 1 : ph);
          }
          const uint32_t t_sfa = tmem_base + SF_COL0 + kpar * 16;
          const uint32_t t_sfb = t_sfa + 4;
          const uint64_t sfd = sfdesc0 + (uint64_t)((s * L::SF_BYTES) >> 4);
          tmem_cp_32x128b_warpx4(t_sfa, sfd);
#pragma unroll
          for (int j = 0; j < NB; ++j) tmem_cp_32x128b_warpx4(t_sfb + 4 * j, sfd + (uint64_t)((512 + j * 512) >> 4));
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          umma_mxf8_ss(tmem_d, ad, bd, idesc[0], t_sfa, t_sfb, accum);
          umma_mxf8_ss(tmem_d, ad + 2, bd + 2, idesc[1], t_sfa, t_sfb, 1u);
          umma_mxf8_ss(tmem_d, ad + 4, bd + 4, idesc[2], t_sfa, t_sfb, 1u);
          umma_mxf8_ss(tmem_d, ad + 6, bd + 6, idesc[3], t_sfa, t_sfb, 1u);
          accum = 1u;
          umma_commit_a(empty_a + s * 8);
          kpar ^= 1;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) umma_commit_a(tfull_a + acc * 8);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int q = warp & 3;
    void* const c = p.c;
    const long long ldc = p.ldc;
    const int m = p.m, n = p.n;
    const uint32_t tempty_a = smem_u32(tempty);
    uint32_t tcount = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++tcount) {
      const TileCoord t = unit_to_tile(unit, 1, group_m, tiles_m, tiles_n);
      const int m0 = t.pid_m * MX_BM, n0 = t.pid_n * BN;
      const uint32_t acc = tcount % NACC;
      const uint32_t aph = (tcount / NACC) & 1;
      if (!mbar_wait(&tfull[acc], aph, status, WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      // two tensor-memory loads in flight; the accumulator is handed back as soon as the last load has landed
      // (before that chunk is converted and stored): the single accumulator's drain is exposed time
      static_assert(BN % 64 == 0, "the drain works on pairs of 32-column chunks");
      uint32_t v0[32], v1[32];
      tmem_ld_32x32b_x32(taddr, v0);
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 64) {
        tmem_ld_wait();
        tmem_ld_32x32b_x32(taddr + cc + 32, v1);
        store_chunk(c, nullptr, ldc, m, n, 0, v0, row, n0 + cc, 0, 1.0f);
        tmem_ld_wait();
        if (cc + 64 < BN) {
          tmem_ld_32x32b_x32(taddr + cc + 64, v0);
        } else {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_a(tempty_a + acc * 8);
        }
        store_chunk(c, nullptr, ldc, m, n, 0, v1, row, n0 + cc + 32, 0, 1.0f);
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

template <int BN, int STAGES>
static int launch_mx(const MxParams& p, int grid, cudaStream_t stream) {
  using L = MxSmem<BN, STAGES>;
  auto kfn = gemm_mxfp8_kernel<BN, STAGES>;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  kfn<<<grid, MX_THREADS, L::TOTAL, stream>>>(p);
  return cuda_err(cudaGetLastError());
}


// --------------------------------------------------------------------------- CTA-pair variant
// 256 x 256 tile per 2-CTA cluster (tcgen05 cta_group::2): CTA r stages A rows [m0+128r, +128) with
// their scale atom, B rows [n0+128r, +128), and the scale atoms of ALL 256 B rows (each CTA's
// tensor core scales its 128 x 256 slice of the accumulator, so it needs every column's scale).
// Per CTA a K step lands 33.5 KB instead of 49.5 KB, which takes the TMA engine off the critical
// path. Scales travel as 2-row boxes of a [atoms*2, 256]-byte tensor map so that, like the operand
// loads, the peer's bytes can be counted on the leader's barrier. One 256-column accumulator plus
// the scale columns fill tensor memory, so the epilogue is not overlapped with the next tile. (Eight epilogue warps
// that take the accumulator into registers with four loads in flight and release it before storing - what brought
// the fp8 x MXFP4 grouped kernel from 2.39 to 1.86 ms - change nothing here: 0.482 ms either way at 8192^3, the
// drain of 14 tiles per cluster being ~2 % of 64 K steps each.)
struct MxPairParams {
  CUtensorMap tma, tmb, tmsa, tmsb;
  void* c;
  int* status;
  long long ldc;
  int m, n;
  int tiles_m, tiles_n, units;
  int k_blocks, n_blocks;
  int group_m;
};

template <int STAGES>
struct MxPairSmem {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = 128 * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // own SFA atom (512 B) + both SFB atoms as one 128-row x 32-byte matrix (4 KB): row L = the 16 bytes of row
  // L % 32 of each atom, in 8-row core groups [group][atom][8 rows x 16 B], so that ONE tcgen05.cp.128x256b fills the
  // eight SFB columns (a scale copy costs ~57 tensor-pipe cycles that do not overlap the MMAs: measured 773 cycles
  // per K step with three copies, 716 with two). Taking the copies off the tensor pipe altogether was tried: four
  // extra warps per CTA read the atoms from shared memory and wrote the scale columns with tcgen05.st (one 16-column
  // store per K step and lane quarter, a barrier per stage towards the MMA thread, with the scale ring on the
  // operand stages and then as a 16-deep ring of its own): 1360-1430 TFLOP/s against 2240-2300 in the same runs -
  // a tcgen05.st issued while MMAs stream takes about a K step's time to complete, so the stores, not the copies,
  // became the critical path.
  static constexpr int SF_BYTES = 512 + 4096;
  static constexpr int SF_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = SF_OFFSET + STAGES * SF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <int STAGES>
__global__ void __launch_bounds__(MX_THREADS, 1) gemm_mxfp8_pair_kernel(const __grid_constant__ MxPairParams p) {
  using L = MxPairSmem<STAGES>;
  constexpr int BN = 256;
  constexpr uint32_t SF_COL0 = BN;
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
  const uint32_t rank = cluster_ctarank();
  const int worker = blockIdx.x >> 1, num_workers = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma);
    tma_prefetch_desc(&p.tmb);
    tma_prefetch_desc(&p.tmsa);
    tma_prefetch_desc(&p.tmsb);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tempty[0], 8);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int units = p.units, group_m = p.group_m, tiles_m = p.tiles_m, tiles_n = p.tiles_n;
  const int k_blocks = p.k_blocks, n_blocks = p.n_blocks;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      const uint32_t leader_full = mapa_shared(full_a, 0);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = worker; unit < units && ok; unit += num_workers) {
        const TileCoord t = unit_to_tile(unit, 1, group_m, tiles_m, tiles_n);
        const int mb = t.pid_m * 2 + (int)rank;          // 128-row block of A staged by this CTA
        const int nb0 = t.pid_n * 2;                     // first 128-row block of B of the tile
        const int m0 = mb * 128, n0 = (nb0 + (int)rank) * 128;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx_a(full_a + s * 8, 2 * (L::STAGE_BYTES + L::SF_BYTES));
          const uint32_t bar = leader_full + s * 8;
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          const uint32_t sf = smem_a + L::SF_OFFSET + s * L::SF_BYTES;
          // out-of-range row blocks (ragged last tile) are zero-filled by the tensor maps
          tma_load_2d_pair(sa, &p.tma, bar, kb * 128, m0, pol);
          tma_load_2d_pair(sa + L::A_BYTES, &p.tmb, bar, kb * 128, n0, pol);
          tma_load_2d_pair(sf, &p.tmsa, bar, 0, 2 * (mb * k_blocks + kb), pol);
          // both SFB atoms, interleaved by 8-row group, once per 32-lane quarter (the copy does not broadcast)
#pragma unroll
          for (int rep4 = 0; rep4 < 4; ++rep4)
            tma_load_4d_pair(sf + 512 + rep4 * 1024, &p.tmsb, bar, 0, nb0, 0, kb, pol);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      (void)n_blocks;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      uint32_t idesc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) idesc[k] = make_idesc_mx(0u, 0u, 256, BN, (uint32_t)k, (uint32_t)k);
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, 16, 1024, SWIZZLE_128B);
      const uint64_t sfdesc0 = make_smem_desc(smem_a + L::SF_OFFSET, 16, 128, SWIZZLE_NONE);
      // SFB matrix: 16 groups of 8 rows, 256 bytes apart; the two 16-byte column blocks of a group 128 bytes apart
      const uint64_t sfbd = make_smem_desc(smem_a + L::SF_OFFSET + 512, 128, 256, SWIZZLE_NONE);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      const uint32_t peer_delta = mapa_shared(empty_a, 1) - empty_a;
      uint32_t s = 0, ph = 0, tcount = 0, kpar = 0;
      bool ok = true, ready = false;
      for (int unit = worker; unit < units && ok; unit += num_workers, ++tcount) {
        if (!mbar_wait_a(tempty_a, (tcount & 1) ^ 1, status, WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base;
        uint32_t accum = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready && !mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          {  // probe the next stage ahead of this stage's MMAs (a blocking wait costs ~70 cycles even when ready)
            const uint32_t s1 = (s + 1 == STAGES) ? 0 : s + 1;
            ready = mbar_test_a(full_a + s1 * 8, s1 == 0 ? ph ^ 1 : ph);
          }
          const uint32_t t_sfa = tmem_base + SF_COL0 + kpar * 16;
          const uint32_t t_sfb = t_sfa + 4;
          const uint64_t sfd = sfdesc0 + (uint64_t)((s * L::SF_BYTES) >> 4);
          tmem_cp_32x128b_warpx4_pair(t_sfa, sfd);
          tmem_cp_128x256b_pair(t_sfb, sfbd + (uint64_t)((s * L::SF_BYTES) >> 4));
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          umma_mxf8_ss_pair(tmem_d, ad, bd, idesc[0], t_sfa, t_sfb, accum);
          umma_mxf8_ss_pair(tmem_d, ad + 2, bd + 2, idesc[1], t_sfa, t_sfb, 1u);
          umma_mxf8_ss_pair(tmem_d, ad + 4, bd + 4, idesc[2], t_sfa, t_sfb, 1u);
          umma_mxf8_ss_pair(tmem_d, ad + 6, bd + 6, idesc[3], t_sfa, t_sfb, 1u);
          accum = 1u;
          umma_commit_pair(empty_a + s * 8);
          umma_commit_pair(empty_a + s * 8 + peer_delta);
          kpar ^= 1;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) {
          umma_commit_pair(tfull_a);
          umma_commit_pair(tfull_a + peer_delta);
        }
      }
    }
  } else {
    const int q = warp & 3;
    void* const c = p.c;
    const long long ldc = p.ldc;
    const int m = p.m, n = p.n;
    const uint32_t tempty_leader = mapa_shared(smem_u32(tempty), 0);
    uint32_t tcount = 0;
    for (int unit = worker; unit < units; unit += num_workers, ++tcount) {
      const TileCoord t = unit_to_tile(unit, 1, group_m, tiles_m, tiles_n);
      const int m0 = (t.pid_m * 2 + (int)rank) * 128, n0 = t.pid_n * BN;
      if (!mbar_wait(&tfull[0], tcount & 1, status, WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
      uint32_t v0[32], v1[32];
      tmem_ld_32x32b_x32(taddr, v0);
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 64) {
        tmem_ld_wait();
        tmem_ld_32x32b_x32(taddr + cc + 32, v1);
        store_chunk(c, nullptr, ldc, m, n, 0, v0, row, n0 + cc, 0, 1.0f);
        tmem_ld_wait();
        if (cc + 64 < BN) {
          tmem_ld_32x32b_x32(taddr + cc + 64, v0);
        } else {  // the last load has landed: hand the accumulator back before the last chunk is stored
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader);
        }
        store_chunk(c, nullptr, ldc, m, n, 0, v1, row, n0 + cc + 32, 0, 1.0f);
      }
    }
  }

  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

static int launch_mx_pair(const tb200_gemm_mxfp8_args* a, int sms, cudaStream_t stream) {
  constexpr int STAGES = 6;
  using L = MxPairSmem<STAGES>;
  MxPairParams p;
  memset(&p, 0, sizeof(p));
  const int k_blocks = (int)(a->k / 128);
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->m};
    const uint64_t strides[1] = {(uint64_t)a->k};
    const uint32_t box[2] = {128, 128};
    int rc = encode_tmap(&p.tma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    const uint64_t dimsb[2] = {(uint64_t)a->k, (uint64_t)a->n};
    rc = encode_tmap(&p.tmb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->b, dimsb, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    // scale atoms as rows of 256 bytes, two rows per atom
    const uint32_t box[2] = {256, 2};
    const uint64_t strides[1] = {256};
    const uint64_t dims_a[2] = {256, (uint64_t)(a->m / 128) * k_blocks * 2};
    const uint64_t dims_b[2] = {256, (uint64_t)(a->n / 128) * k_blocks * 2};
    int rc = encode_tmap(&p.tmsa, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a_scale, dims_a, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TB200_OK) return rc;
    (void)dims_b;
    // B scales: (128 bytes of an 8-row group, atom's N block, group in the atom, K block); a box of two N blocks x
    // four groups lands as [group][N block][128 bytes] = 32 rows of the matrix the 128x256b copy reads
    const uint64_t dims4[4] = {128, (uint64_t)(a->n / 128), 4, (uint64_t)k_blocks};
    const uint64_t strides4[3] = {(uint64_t)k_blocks * 512, 128, 512};
    const uint32_t box4[4] = {128, 2, 4, 1};
    rc = encode_tmap(&p.tmsb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->b_scale, dims4, strides4, box4, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TB200_OK) return rc;
  }
  p.c = a->c;
  p.ldc = a->ldc;
  p.m = (int)a->m;
  p.n = (int)a->n;
  p.tiles_m = (int)((a->m + 255) / 256);
  p.tiles_n = (int)((a->n + 255) / 256);
  p.units = p.tiles_m * p.tiles_n;
  p.k_blocks = k_blocks;
  p.n_blocks = (int)(a->n / 128);
  p.group_m = 8;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  auto kfn = gemm_mxfp8_pair_kernel<STAGES>;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  const int clusters = p.units < sms / 2 ? p.units : sms / 2;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(MX_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_err(cudaLaunchKernelEx(&cfg, kfn, p));
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_gemm_mxfp8(const tb200_gemm_mxfp8_args* a, void* stream_) {
  if (!a || !a->a || !a->b || !a->c || !a->a_scale || !a->b_scale) return TB200_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return (a->m == 0 || a->n == 0) ? TB200_OK : TB200_ERR_BAD_ARG;
  if ((a->m % 128) || (a->n % 128) || (a->k % 128)) return TB200_ERR_UNSUPPORTED;
  if (a->m > INT32_MAX || a->n > INT32_MAX || a->k > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15) ||
      (reinterpret_cast<uintptr_t>(a->a_scale) & 15) || (reinterpret_cast<uintptr_t>(a->b_scale) & 15))
    return TB200_ERR_BAD_ARG;
  if (a->ldc < a->n) return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  {
    const long long t256 = ((a->m + 255) / 256) * ((a->n + 255) / 256);
    (void)t256;  // the pair tiling measures the same as the single-CTA one at 8192^3 (2325 / 2318 TFLOP/s): on request only
    if (a->block_n == 512) return launch_mx_pair(a, sms, stream);
  }
  MxParams p;
  memset(&p, 0, sizeof(p));
  int bn = a->block_n;
  if (bn == 0) {
    // 256-wide tiles once they fill the machine, else 128-wide ones (twice as many tiles)
    const long long t256 = (a->m / 128) * ((a->n + 255) / 256);
    bn = (t256 >= sms) ? 256 : 128;
  }
  if (bn != 128 && bn != 256) return TB200_ERR_UNSUPPORTED;
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->m};
    const uint64_t strides[1] = {(uint64_t)a->k};
    const uint32_t box[2] = {128, 128};
    int rc = encode_tmap(&p.tma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->n};
    const uint64_t strides[1] = {(uint64_t)a->k};
    const uint32_t box[2] = {128, (uint32_t)bn};
    int rc = encode_tmap(&p.tmb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.sfa = static_cast<const uint8_t*>(a->a_scale);
  p.sfb = static_cast<const uint8_t*>(a->b_scale);
  p.c = a->c;
  p.ldc = a->ldc;
  p.m = (int)a->m;
  p.n = (int)a->n;
  p.k = (int)a->k;
  p.tiles_m = (int)(a->m / 128);
  p.tiles_n = (int)((a->n + bn - 1) / bn);
  p.units = p.tiles_m * p.tiles_n;
  p.k_blocks = (int)(a->k / 128);
  p.n_blocks = (int)(a->n / 128);
  p.group_m = 8;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  const int grid = p.units < sms ? p.units : sms;
  return bn == 256 ? launch_mx<256, 4>(p, grid, stream) : launch_mx<128, 6>(p, grid, stream);
}
