// Grouped (per-expert) GEMM with FP8 activations and MXFP4 weights for sm_100a:
//
//   for each expert e and each sorted row r in [slice_offs[e], slice_offs[e+1]):
//       acc      = x_scale * X[r, :] @ dequant(W[e])   (+ bias[e])       W[e][n, k] = e2m1 * 2^(scale[n, k/32] - 127)
//       acc      = swiglu(acc)                          (optional)
//       Y[scatter[r], :] = acc * gammas[r]
//
// X [rows, K] is e4m3 (or e5m2), rows sorted by expert; W holds two e2m1 values per byte along K (low nibble
// first), blocked as [E][N/256][K/128][256 rows][64 bytes] so that what one tile needs per K step is one
// contiguous 16 KB run (with 64-byte pieces of 256 different rows the same kernel reached 40 % of the HBM
// rate), with one e8m0 scale per 32 values of K, stored per expert in the 512-byte
// atom order of the MXFP8 kernel ([n/128][K/128][n%32][n/32%4][k%4]). The weights stay packed in HBM
// (4.25 bits per value: the decode regime streams 3.8x fewer bytes than bf16); the TMA unpacks them on
// the way into shared memory (tensor-map type 16U4_ALIGN16B: 16 values in 8 bytes + 8 bytes of padding,
// the operand format tcgen05.mma.kind::mxf8f6f4 wants for 4-bit types), so a K step of 128 values is a
// 128-byte row like an fp8 one and the MMA loop is that of the MXFP8 kernel: scale atoms copied to
// tensor memory with tcgen05.cp, four block-scaled MMAs of K = 32 per step. The activations carry no
// block scales: their scale columns are written once with 1.0 (0x7f).
// Work units are (block-schedule entry, N tile) as in the bf16 grouped kernel; one 128 x 256 accumulator
// plus the scale columns fill tensor memory. Roles (320 threads): TMA warp, MMA warp, 8 epilogue warps, which
// take the accumulator into registers and hand tensor memory back before they compute and store.
// (Handing the accumulator over in two 128-column halves, as the dense wide tile does - the first and last one or
// two K steps of a tile issued as N = 128 MMAs on one half while the other half is drained - measured equal with one
// split step each end and 4 % slower with two: the split steps read the activation tile twice and copy more scales,
// which costs what the shorter hand-over saves.)
// With a few rows per expert (decode) this kernel streams the weights at 2.9 TB/s: per K step the four
// 128 x 256 MMAs cost ~530 cycles however few rows are real, and the single accumulator serialises the
// epilogue. A variant that moved the weights packed through an 8-deep ring and unpacked them with the
// epilogue warps (twice the bytes in flight) measured slower (2.6 TB/s: its loads were never late, the
// unpacking took ~700 cycles per step next to the MMAs' operand traffic); swapping the operand roles (weight
// rows on the MMA's M, tokens on a small N) is what the second kernel below does (3.1-3.4 TB/s; with 72 KB
// of packed weights in flight per SM it is bound by load latency, and the padded operand format costs two
// bytes of shared memory per byte in flight).
//
// Counterpart in the reference: _p_matmul with an mxfp4 weight (python/triton_kernels/triton_kernels/
// matmul_details/_p_matmul.py: scaled dot :466-530), host entry triton_kernels/matmul.py:243 with
// PrecisionConfig(weight_scale=...); weight preparation bench/bench_mlp.py:36-57.
#include <string.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "host_common.h"
#include "moe_epilogue.cuh"

namespace tb200 {

static constexpr int M4_THREADS = 192;
static constexpr int M4_BIG_THREADS = 320;  // the many-rows kernel: TMA warp, MMA warp, 8 epilogue warps
static constexpr int M4_BM = 128;
static constexpr int M4_BN = 256;
static constexpr int M4_STAGES = 4;

struct Mx4Params {
  CUtensorMap tmx;  // X: (K bytes, rows), box (128, 128), fp8 as bytes
  CUtensorMap tmw;  // W blocks: (128 values, rows) 16U4_ALIGN16B, box (128, 256)
  const uint8_t* sfw;  // [E][N/128][K/128][512]
  const int* slice_offs;
  const int* slice_sizes;
  const int* sched;
  const int* scatter;
  const float* gammas;
  const float* bias;
  const float* x_scale;  // optional: one float, multiplies every accumulator
  const float* w_flex;   // optional: one float, the weight's flexpoint scale (multiplies every accumulator too)
  const float* y_expected;  // optional flexpoint output: the result is divided by this value ...
  float* y_actual;          // ... and max |result| / max_finite(out type) is folded into this one with an atomic max
  int saturate;             // clamp the scaled output to the finite range of the output type
  const uint8_t* x_sf;   // optional e8m0 block scales of the activations: [rows_x][K/32], ld_xsf bytes between rows
  uint8_t* y_sf;         // optional: the output is MX-quantised, its e8m0 scales go to [rows_y][N_out/32] (ld_ysf)
  long long ld_xsf, ld_ysf;
  void* y;
  int* status;
  long long ldy;
  int n_sched, tiles_n, units;
  int n, k_blocks, n_blocks, rows_x, rows_y;
  int swiglu, has_limit, out_kind;
  float alpha, limit;
  uint32_t idesc[4];
};

struct Mx4Smem {
  static constexpr int A_BYTES = M4_BM * 128;
  static constexpr int B_BYTES = M4_BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SF_BYTES = 3 * 512;  // two scale atoms of W per K step + one of the activations (MX-scaled x)
  static constexpr int SF_OFFSET = M4_STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = SF_OFFSET + M4_STAGES * SF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * M4_STAGES + 2) * 8 + 16 + 1024;
};

// EXT: the instantiation with MX-scaled activations, MX-quantised output and flexpoint scales; the plain one compiles
// them out, which keeps its producer and epilogue loops as short as they were before those existed (4-8 % of a layer).
// WF8: the weights are fp8 bytes ([E][N][K], K contiguous) behind a three-dimensional tensor map instead of packed
// e2m1 blocks; their scale atoms are optional (none: plain fp8 weights, scale columns of 1.0; given: MXFP8 weights).
template <bool EXT, bool WF8>
__global__ void __launch_bounds__(M4_BIG_THREADS, 1) moe_gemm_mx4_kernel(const __grid_constant__ Mx4Params p) {
  using L = Mx4Smem;
  constexpr int BN = M4_BN, STAGES = M4_STAGES;
  constexpr uint32_t SFA_COL = 256;       // four columns of 1.0 for the activations
  constexpr uint32_t SFW_COL0 = 256 + 16; // two sets of 8 columns for the weight scales
  constexpr uint32_t SFX_COL0 = 256 + 32; // two sets of 4 columns for the activations' own block scales
  constexpr uint32_t SFW_ONE = 256 + 48;  // eight columns of 1.0 for weights without block scales
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 1);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmx);
    tma_prefetch_desc(&p.tmw);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, 8);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  if (warp >= 2 && warp < 6) {  // activation scale columns: 1.0 in every byte, on all 128 lanes
    const uint32_t one = 0x7f7f7f7fu;
    tmem_st_32x32b_x4(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SFA_COL, one, one, one, one);
    if (WF8) {
      tmem_st_32x32b_x4(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SFW_ONE, one, one, one, one);
      tmem_st_32x32b_x4(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SFW_ONE + 4, one, one, one, one);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const int units = p.units, tiles_n = p.tiles_n, k_blocks = p.k_blocks, n_blocks = p.n_blocks;
  const int* const sched = p.sched;
  const int* const slice_offs = p.slice_offs;
  const int* const slice_sizes = p.slice_sizes;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    // One lane issues the bulk copies. With MX-scaled activations the whole warp takes part: lane l fetches the four
    // scale bytes of this K step for rows l, l + 32, l + 64, l + 96 (one step ahead, so the loads are in flight
    // while the warp waits for a free stage) and writes them as the 16 bytes of row l of a 512-byte atom
    // ([row % 32][row / 32][k]), the order tcgen05.cp.32x128b.warpx4 turns into the MMA's scale columns.
    const uint8_t* const x_sf = EXT ? p.x_sf : nullptr;
    if (lane == 0 || x_sf) {
      // both kept in L2: a weight tile is read by the expert's other row blocks a few units later, an activation
      // block by the other column tiles (the 16384-token layer with evict_first weights / evict_normal activations
      // 1.86 ms, evict_last weights 1.80, both evict_last 1.75-1.78; with fp8 weights 2.11 / 2.00 / 1.93)
      const uint64_t pol_x = policy_evict_last();
      const uint64_t pol_w = policy_evict_last();
      const long long ld_xsf = p.ld_xsf;
      const int rows_x = p.rows_x;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const int si = unit / tiles_n;
        const int entry = __ldg(sched + si);
        if (entry < 0) continue;
        const int e = entry & 0xFFFF;
        const int pid_n = unit - si * tiles_n;
        const int n0 = pid_n * BN;
        const int row0 = __ldg(slice_offs + e) + (entry >> 16) * M4_BM;
        const int nb_valid = min(2, n_blocks - pid_n * 2);
        const uint8_t* atoms = p.sfw + ((size_t)e * n_blocks + (size_t)pid_n * 2) * k_blocks * 512;
        uint32_t sfx[4] = {0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu};
        auto load_sfx = [&](int kb) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = row0 + lane + 32 * i;
            sfx[i] = r < rows_x ? __ldg(reinterpret_cast<const uint32_t*>(x_sf + (long long)r * ld_xsf) + kb) : 0x7f7f7f7fu;
          }
        };
        if (x_sf) load_sfx(0);
        for (int kb = 0; kb < k_blocks; ++kb) {
          bool free_stage = true;
          if (lane == 0) free_stage = mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY);
          if (x_sf) free_stage = __shfl_sync(0xffffffffu, free_stage ? 1 : 0, 0) != 0;
          if (!free_stage) {
            ok = false;
            break;
          }
          uint8_t* sf = smem + L::SF_OFFSET + s * L::SF_BYTES;
          if (x_sf) {
            *reinterpret_cast<uint4*>(sf + 1024 + lane * 16) = make_uint4(sfx[0], sfx[1], sfx[2], sfx[3]);
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t bar = full_a + s * 8;
            const uint32_t sa = smem_a + s * L::STAGE_BYTES;
            if (WF8) {
              const bool w_scaled = p.sfw != nullptr;
              mbar_expect_tx_a(bar, L::A_BYTES + L::B_BYTES + (w_scaled ? nb_valid * 512 : 0));
              tma_load_2d_a(sa, &p.tmx, bar, kb * 128, row0, pol_x);
              tma_load_3d(smem + s * L::STAGE_BYTES + L::A_BYTES, &p.tmw, &full[s], kb * 128, n0, e, pol_w);
              if (w_scaled)
                for (int j = 0; j < nb_valid; ++j)
                  bulk_load(sf + j * 512, atoms + ((size_t)j * k_blocks + kb) * 512, 512, &full[s]);
            } else {
              // the unpacking load of W reports the bytes it read (64 per row), not the 128 it writes
              mbar_expect_tx_a(bar, L::A_BYTES + L::B_BYTES / 2 + nb_valid * 512);
              tma_load_2d_a(sa, &p.tmx, bar, kb * 128, row0, pol_x);
              tma_load_2d_a(sa + L::A_BYTES, &p.tmw, bar, 0, (((e * tiles_n + pid_n) * k_blocks) + kb) * BN, pol_w);
              for (int j = 0; j < nb_valid; ++j)
                bulk_load(sf + j * 512, atoms + ((size_t)j * k_blocks + kb) * 512, 512, &full[s]);
            }
          }
          if (x_sf && kb + 1 < k_blocks) load_sfx(kb + 1);
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
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, 16, 1024, SWIZZLE_128B);
      const uint64_t sfdesc0 = make_smem_desc(smem_a + L::SF_OFFSET, 16, 128, SWIZZLE_NONE);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      const uint32_t t_sfa_one = tmem_base + SFA_COL;
      const bool mx_x = EXT && p.x_sf != nullptr;
      const bool w_scaled = !WF8 || p.sfw != nullptr;
      uint32_t s = 0, ph = 0, tcount = 0, kpar = 0;
      bool ok = true, ready = false;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        if (__ldg(sched + unit / tiles_n) < 0) continue;
        if (!mbar_wait_a(tempty_a, (tcount & 1) ^ 1, status, WAIT_TMEM_EMPTY)) break;
        ++tcount;
        tc_fence_after_sync();
        uint32_t accum = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready && !mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s1 = (s + 1 == STAGES) ? 0 : s + 1;
          ready = mbar_test_a(full_a + s1 * 8, s1 == 0 ? ph ^ 1 : ph);
          uint32_t t_sfw = tmem_base + SFW_COL0 + kpar * 8;
          const uint64_t sfd = sfdesc0 + (uint64_t)((s * L::SF_BYTES) >> 4);
          if (WF8 && !w_scaled) {
            t_sfw = tmem_base + SFW_ONE;
          } else {
            tmem_cp_32x128b_warpx4(t_sfw, sfd);
            tmem_cp_32x128b_warpx4(t_sfw + 4, sfd + (uint64_t)(512 >> 4));
          }
          uint32_t t_sfa = t_sfa_one;
          if (mx_x) {
            t_sfa = tmem_base + SFX_COL0 + kpar * 4;
            tmem_cp_32x128b_warpx4(t_sfa, sfd + (uint64_t)(1024 >> 4));
          }
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          umma_mxf8_ss(tmem_base, ad, bd, p.idesc[0], t_sfa, t_sfw, accum);
          umma_mxf8_ss(tmem_base, ad + 2, bd + 2, p.idesc[1], t_sfa, t_sfw, 1u);
          umma_mxf8_ss(tmem_base, ad + 4, bd + 4, p.idesc[2], t_sfa, t_sfw, 1u);
          umma_mxf8_ss(tmem_base, ad + 6, bd + 6, p.idesc[3], t_sfa, t_sfw, 1u);
          accum = 1u;
          umma_commit_a(empty_a + s * 8);
          kpar ^= 1;
          s = s1;
          if (s == 0) ph ^= 1;
        }
        if (ok) umma_commit_a(tfull_a);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    // Eight warps: warp w reads lanes 32 (w % 4) .. of tensor memory, the first four take columns 0-127 of the tile,
    // the other four 128-255. A thread first moves its 128 accumulator values to registers and releases the
    // accumulator, so the next tile's MMAs run under the arithmetic and the stores of this one (with one accumulator
    // in tensor memory and the epilogue done from there, a third of the layer's GEMM time was epilogue).
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int n = p.n, rows_y = p.rows_y;
    void* const y = p.y;
    const float acc_scale = (p.x_scale ? __ldg(p.x_scale) : 1.f) * (EXT && p.w_flex ? __ldg(p.w_flex) : 1.f);
    MoeEpilogueExtra flex;
    if (EXT && p.y_expected) {
      flex.inv_expected = 1.f / __ldg(p.y_expected);
      if (p.saturate) flex.clip = p.out_kind == MOE_OUT_E5M2 ? 57344.f : p.out_kind == MOE_OUT_E4M3 ? 448.f : 65504.f;
    }
    flex.track_absmax = EXT && p.y_actual != nullptr;
    const uint32_t tempty_a = smem_u32(tempty);
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + (uint32_t)half * 128;
    uint32_t tcount = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const int si = unit / tiles_n;
      const int entry = __ldg(sched + si);
      if (entry < 0) continue;
      const int e = entry & 0xFFFF;
      const int n0 = (unit - si * tiles_n) * BN + half * 128;
      const int row0 = __ldg(slice_offs + e) + (entry >> 16) * M4_BM;
      const int row_end = slice_sizes ? __ldg(slice_offs + e) + __ldg(slice_sizes + e) : __ldg(slice_offs + e + 1);
      const int sr = row0 + q * 32 + lane;
      int out_row = -1;
      float gamma = 1.f;
      if (sr < row_end) {
        out_row = p.scatter ? __ldg(p.scatter + sr) : sr;
        if (out_row >= rows_y) out_row = -1;
        if (p.gammas) gamma = __ldg(p.gammas + sr);
      }
      const float* brow = p.bias ? p.bias + (long long)e * n : nullptr;
      if (!mbar_wait(tfull, tcount & 1, status, WAIT_TMEM_FULL)) break;
      ++tcount;
      tc_fence_after_sync();
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(taddr + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(tempty_a);
      float absmax = 0.f;
      if (out_row >= 0) {
        if (EXT && p.y_sf) {
          // MX-quantised output: a block of 32 outputs is one chunk of 32 accumulator columns, or two with SwiGLU
          if (p.swiglu) {
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
              const int col = n0 + c * 32;
              if (col >= n) break;
              float o[32];
              moe_chunk_values<0>(v[c], col, n, brow, 1, p.alpha, p.limit, p.has_limit, gamma, acc_scale,
                                  MoeEpilogueExtra(), o);
              moe_chunk_values<16>(v[c + 1], col + 32, n, brow, 1, p.alpha, p.limit, p.has_limit, gamma, acc_scale,
                                   MoeEpilogueExtra(), o);
              const int ocol = col >> 1;
              moe_store_mx_block(o, min(32, (n - col) >> 1), y, (long long)out_row * p.ldy + ocol,
                                 p.y_sf + (long long)out_row * p.ld_ysf + (ocol >> 5), p.out_kind);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int col = n0 + c * 32;
              if (col >= n) break;
              float o[32];
              moe_chunk_values<0>(v[c], col, n, brow, 0, p.alpha, p.limit, p.has_limit, gamma, acc_scale,
                                  MoeEpilogueExtra(), o);
              moe_store_mx_block(o, min(32, n - col), y, (long long)out_row * p.ldy + col,
                                 p.y_sf + (long long)out_row * p.ld_ysf + (col >> 5), p.out_kind);
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int col = n0 + c * 32;
            if (col >= n) break;
            absmax = fmaxf(absmax, moe_store_chunk(v[c], y, p.ldy, out_row, col, n, brow, p.swiglu, p.alpha, p.limit,
                                                   p.has_limit, gamma, p.out_kind, acc_scale, flex));
          }
        }
      }
      if (EXT && p.y_actual && !p.y_sf) moe_flex_publish(absmax, p.y_actual, p.out_kind);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// --------------------------------------------------------------------------- few rows per expert
// Operand roles swapped: the MMA's M = 128 weight rows (A: the unpacked weight tile, its e8m0 atom as the A
// scales), N = 32 token rows (B: a 32-row activation tile of the 32-row block schedule, scales 1.0). A K
// step then costs four N = 32 MMAs (~46 cycles each) per 128 weight rows instead of four 128 x 256 ones
// (~530 cycles per 256 rows), a stage is 20.5 KB (9 of them), and a 128 x 32 accumulator is 32 columns, so
// four of them rotate and the epilogue never blocks the MMAs. The accumulator is the output transposed:
// thread = weight row n, columns = tokens; a warp writes 32 consecutive n of one token (64 bytes), SwiGLU
// pairs are adjacent lanes.
static constexpr int S4_XROWS = 32;
static constexpr int S4_WROWS = 128;
static constexpr int S4_STAGES = 9;
static constexpr int S4_NACC = 4;

struct Mx4SwapSmem {
  static constexpr int W_BYTES = S4_WROWS * 128;  // unpacked
  static constexpr int X_BYTES = S4_XROWS * 128;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;  // 20 KB, a multiple of 1024
  static constexpr int SF_OFFSET = S4_STAGES * STAGE_BYTES;
  static constexpr int SF_BYTES = 2 * 512;  // the weight tile's scale atom + one for MX-scaled activations
  static constexpr int BAR_OFFSET = SF_OFFSET + S4_STAGES * SF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * S4_STAGES + 2 * S4_NACC) * 8 + 16 + 1024;
};
static_assert(Mx4SwapSmem::TOTAL <= 232448, "shared memory budget");

template <bool EXT>
__global__ void __launch_bounds__(M4_THREADS, 1) moe_gemm_mx4_swap_kernel(const __grid_constant__ Mx4Params p) {
  using L = Mx4SwapSmem;
  constexpr int STAGES = S4_STAGES;
  constexpr uint32_t SFB_COL = S4_NACC * 32;      // token-side scale columns: 1.0
  constexpr uint32_t SFA_COL0 = SFB_COL + 8;      // two sets of 4 columns for the weight scales
  constexpr uint32_t SFX_COL0 = SFB_COL + 16;     // two sets of 4 columns for the tokens' own block scales
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;   // [NACC]
  uint64_t* tempty = tfull + S4_NACC; // [NACC] 4 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + S4_NACC);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tmx);
    tma_prefetch_desc(&p.tmw);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < S4_NACC; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  if (warp >= 2) {
    const uint32_t one = 0x7f7f7f7fu;
    tmem_st_32x32b_x4(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SFB_COL, one, one, one, one);
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  // units: (entry of the 32-row schedule, tile of 128 weight rows)
  const int units = p.units, tiles_w = p.tiles_n, k_blocks = p.k_blocks, n_blocks = p.n_blocks;
  const int tiles_256 = (n_blocks + 1) / 2;  // 256-row blocks of the weight buffer per (expert, K step)
  const int* const sched = p.sched;
  const int* const slice_offs = p.slice_offs;
  const int* const slice_sizes = p.slice_sizes;
  int* const status = p.status;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    // With MX-scaled activations lane l also stages the four scale bytes of token row0 + l for each K step (row l of
    // a 512-byte atom, the other twelve bytes of the row are 1.0), fetched one step ahead.
    const uint8_t* const x_sf = EXT ? p.x_sf : nullptr;
    if (lane == 0 || x_sf) {
      const uint64_t pol_x = policy_evict_last();
      const uint64_t pol_w = policy_evict_first();
      const long long ld_xsf = p.ld_xsf;
      const int rows_x = p.rows_x;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const int si = unit / tiles_w;
        const int entry = __ldg(sched + si);
        if (entry < 0) continue;
        const int e = entry & 0xFFFF;
        const int wt = unit - si * tiles_w;  // 128-row weight tile
        const int row0 = __ldg(slice_offs + e) + (entry >> 16) * S4_XROWS;
        const uint8_t* atoms = p.sfw + ((size_t)e * n_blocks + wt) * k_blocks * 512;
        // weight rows 128 wt .. of expert e sit in 256-row block wt / 2, half wt % 2, of each K step
        const int wrow0 = ((e * tiles_256 + (wt >> 1)) * k_blocks) * M4_BN + (wt & 1) * S4_WROWS;
        uint32_t sfx = 0x7f7f7f7fu;
        auto load_sfx = [&](int kb) {
          const int r = row0 + lane;
          sfx = r < rows_x ? __ldg(reinterpret_cast<const uint32_t*>(x_sf + (long long)r * ld_xsf) + kb) : 0x7f7f7f7fu;
        };
        if (x_sf) load_sfx(0);
        for (int kb = 0; kb < k_blocks; ++kb) {
          bool free_stage = true;
          if (lane == 0) free_stage = mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY);
          if (x_sf) free_stage = __shfl_sync(0xffffffffu, free_stage ? 1 : 0, 0) != 0;
          if (!free_stage) {
            ok = false;
            break;
          }
          uint8_t* sf = smem + L::SF_OFFSET + s * L::SF_BYTES;
          if (x_sf) {
            *reinterpret_cast<uint4*>(sf + 512 + lane * 16) = make_uint4(sfx, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t bar = full_a + s * 8;
            mbar_expect_tx_a(bar, L::W_BYTES / 2 + L::X_BYTES + 512);
            const uint32_t sw = smem_a + s * L::STAGE_BYTES;
            tma_load_2d_a(sw, &p.tmw, bar, 0, wrow0 + kb * M4_BN, pol_w);
            tma_load_2d_a(sw + L::W_BYTES, &p.tmx, bar, kb * 128, row0, pol_x);
            bulk_load(sf, atoms + (size_t)kb * 512, 512, &full[s]);
          }
          if (x_sf && kb + 1 < k_blocks) load_sfx(kb + 1);
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
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::W_BYTES, 16, 1024, SWIZZLE_128B);
      const uint64_t sfdesc0 = make_smem_desc(smem_a + L::SF_OFFSET, 16, 128, SWIZZLE_NONE);
      const uint32_t tfull_a = smem_u32(tfull), tempty_a = smem_u32(tempty);
      const uint32_t t_sfb_one = tmem_base + SFB_COL;
      const bool mx_x = EXT && p.x_sf != nullptr;
      uint32_t s = 0, ph = 0, tcount = 0, kpar = 0;
      bool ok = true, ready = false;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        if (__ldg(sched + unit / tiles_w) < 0) continue;
        const uint32_t acc = tcount % S4_NACC, aph = (tcount / S4_NACC) & 1;
        ++tcount;
        if (!mbar_wait_a(tempty_a + acc * 8, aph ^ 1, status, WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * 32;
        uint32_t accum = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready && !mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s1 = (s + 1 == STAGES) ? 0 : s + 1;
          ready = mbar_test_a(full_a + s1 * 8, s1 == 0 ? ph ^ 1 : ph);
          const uint32_t t_sfa = tmem_base + SFA_COL0 + kpar * 4;
          tmem_cp_32x128b_warpx4(t_sfa, sfdesc0 + (uint64_t)((s * L::SF_BYTES) >> 4));
          uint32_t t_sfb = t_sfb_one;
          if (mx_x) {
            t_sfb = tmem_base + SFX_COL0 + kpar * 4;
            tmem_cp_32x128b_warpx4(t_sfb, sfdesc0 + (uint64_t)((s * L::SF_BYTES + 512) >> 4));
          }
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          umma_mxf8_ss(tmem_d, ad, bd, p.idesc[0], t_sfa, t_sfb, accum);
          umma_mxf8_ss(tmem_d, ad + 2, bd + 2, p.idesc[1], t_sfa, t_sfb, 1u);
          umma_mxf8_ss(tmem_d, ad + 4, bd + 4, p.idesc[2], t_sfa, t_sfb, 1u);
          umma_mxf8_ss(tmem_d, ad + 6, bd + 6, p.idesc[3], t_sfa, t_sfb, 1u);
          accum = 1u;
          umma_commit_a(empty_a + s * 8);
          kpar ^= 1;
          s = s1;
          if (s == 0) ph ^= 1;
        }
        if (ok) umma_commit_a(tfull_a + acc * 8);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (transposed accumulator)
    const int q = warp & 3;
    const int n = p.n, rows_y = p.rows_y, swiglu = p.swiglu, has_limit = p.has_limit, out_kind = p.out_kind;
    const float alpha = p.alpha, limit = p.limit;
    void* const y = p.y;
    const long long ldy = p.ldy;
    const float acc_scale = (p.x_scale ? __ldg(p.x_scale) : 1.f) * (EXT && p.w_flex ? __ldg(p.w_flex) : 1.f);
    const float inv_expected = EXT && p.y_expected ? 1.f / __ldg(p.y_expected) : 1.f;
    const float clip = (EXT && p.y_expected && p.saturate)
                           ? (out_kind == MOE_OUT_E5M2 ? 57344.f : out_kind == MOE_OUT_E4M3 ? 448.f : 65504.f) : 0.f;
    float* const y_actual = EXT ? p.y_actual : nullptr;
    uint8_t* const y_sf = EXT ? p.y_sf : nullptr;
    const long long ld_ysf = p.ld_ysf;
    const uint32_t tempty_a = smem_u32(tempty);
    uint32_t tcount = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const int si = unit / tiles_w;
      const int entry = __ldg(sched + si);
      if (entry < 0) continue;
      const int e = entry & 0xFFFF;
      const int wt = unit - si * tiles_w;
      const int row0 = __ldg(slice_offs + e) + (entry >> 16) * S4_XROWS;
      const int row_end = slice_sizes ? __ldg(slice_offs + e) + __ldg(slice_sizes + e) : __ldg(slice_offs + e + 1);
      const int valid = min(S4_XROWS, row_end - row0);
      const uint32_t acc = tcount % S4_NACC, aph = (tcount / S4_NACC) & 1;
      ++tcount;
      if (!mbar_wait(&tfull[acc], aph, status, WAIT_TMEM_FULL)) break;
      tc_fence_after_sync();
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * 32, v);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(tempty_a + acc * 8);  // the accumulator is in registers
      const int col = wt * S4_WROWS + q * 32 + lane;  // weight row = output column of this thread
      const float b = (p.bias && col < n) ? __ldg(p.bias + (long long)e * n + col) : 0.f;
      float absmax = 0.f;
#pragma unroll
      for (int c = 0; c < S4_XROWS; ++c) {
        if (c >= valid) break;
        const int sr = row0 + c;
        int out_row = p.scatter ? __ldg(p.scatter + sr) : sr;
        if (out_row >= rows_y) out_row = -1;
        const float gamma = p.gammas ? __ldg(p.gammas + sr) : 1.f;
        float f = __uint_as_float(v[c]) * acc_scale + b;
        if (y_sf) {
          // MX-quantised output (no SwiGLU here): the warp's 32 columns are one block of this token's row
          const float o = f * gamma;
          float amax = fabsf(o);
#pragma unroll
          for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
          const float max_finite = out_kind == MOE_OUT_E5M2 ? 57344.f : 448.f;
          const uint32_t bits = (__float_as_uint(__fdiv_rn(amax, max_finite)) + 0x007FFFFFu) & 0x7F800000u;
          const float inv = bits == 0u ? 0.f : __frcp_rn(__uint_as_float(bits));
          if (out_row >= 0 && col < n) {
            moe_store_one(y, (long long)out_row * ldy + col, o * inv, out_kind);
            if (lane == 0) y_sf[(long long)out_row * ld_ysf + (col >> 5)] = (uint8_t)(bits >> 23);
          }
          continue;
        }
        if (swiglu) {
          const float other = __shfl_xor_sync(0xffffffffu, f, 1);  // (gate, linear) are adjacent columns
          if ((lane & 1) == 0 && out_row >= 0 && col < n) {
            float o = moe_swiglu(f, other, alpha, limit, has_limit) * gamma;
            absmax = fmaxf(absmax, fabsf(o));
            o *= inv_expected;
            if (clip > 0.f) o = fminf(fmaxf(o, -clip), clip);
            moe_store_one(y, (long long)out_row * ldy + (col >> 1), o, out_kind);
          }
        } else if (out_row >= 0 && col < n) {
          float o = f * gamma;
          absmax = fmaxf(absmax, fabsf(o));
          o *= inv_expected;
          if (clip > 0.f) o = fminf(fmaxf(o, -clip), clip);
          moe_store_one(y, (long long)out_row * ldy + col, o, out_kind);
        }
      }
      if (y_actual && !y_sf) moe_flex_publish(absmax, y_actual, out_kind);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_moe_gemm_mx4(const tb200_moe_gemm_mx4_args* a, void* stream_) {
  if (!a || !a->x || !a->w || !a->y || !a->slice_offs || !a->block_schedule) return TB200_ERR_BAD_ARG;
  const bool wf8 = a->w_dtype == TB200_E4M3 || a->w_dtype == TB200_E5M2;
  if (!wf8 && (a->w_dtype != 0 || !a->w_scale)) return TB200_ERR_BAD_ARG;
  if (a->n_experts <= 0 || a->n_experts > 65535 || a->k <= 0 || a->n <= 0 || a->n_sched < 0) return TB200_ERR_BAD_ARG;
  if (a->rows_x < 0 || a->rows_y < 0) return TB200_ERR_BAD_ARG;
  if (a->x_dtype != TB200_E4M3 && a->x_dtype != TB200_E5M2) return TB200_ERR_UNSUPPORTED;
  if (a->out_dtype != TB200_BF16 && a->out_dtype != TB200_F16 && a->out_dtype != TB200_E4M3 &&
      a->out_dtype != TB200_E5M2)
    return TB200_ERR_UNSUPPORTED;
  if (wf8 ? (a->k % 16) != 0 : (a->k % 32) != 0) return TB200_ERR_UNSUPPORTED;
  if (a->swiglu && (a->n & 1)) return TB200_ERR_BAD_ARG;
  if ((a->ldx % 16) || a->ldx < a->k) return TB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) || (reinterpret_cast<uintptr_t>(a->w) & (wf8 ? 15 : 31)) ||
      (reinterpret_cast<uintptr_t>(a->w_scale) & 15))
    return TB200_ERR_BAD_ARG;
  if (a->rows_x > INT32_MAX - 1 || a->rows_y > INT32_MAX || a->k > INT32_MAX || a->n > INT32_MAX)
    return TB200_ERR_UNSUPPORTED;
  if (a->x_mx_scale && ((reinterpret_cast<uintptr_t>(a->x_mx_scale) & 3) || (a->ld_x_mx_scale % 4) ||
                        a->ld_x_mx_scale < (a->k + 127) / 128 * 4))
    return TB200_ERR_BAD_ARG;
  if (a->y_mx_scale) {
    const int64_t n_out = a->swiglu ? a->n / 2 : a->n;
    if (a->out_dtype != TB200_E4M3 && a->out_dtype != TB200_E5M2) return TB200_ERR_BAD_ARG;
    if (a->ld_y_mx_scale < (n_out + 31) / 32) return TB200_ERR_BAD_ARG;
  }
  if (a->n_sched == 0 || a->rows_x == 0) return TB200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  const bool swap = a->block_rows == S4_XROWS;
  if (!swap && a->block_rows != 0 && a->block_rows != M4_BM) return TB200_ERR_BAD_ARG;
  if (swap && wf8) return TB200_ERR_UNSUPPORTED;  // fp8 weights: the 128-row schedule only
  // the swapped kernel quantises a warp's 32 columns as one block; with SwiGLU a block would span two warps
  if (swap && a->y_mx_scale && a->swiglu) return TB200_ERR_UNSUPPORTED;
  Mx4Params p;
  memset(&p, 0, sizeof(p));
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->rows_x};
    const uint64_t strides[1] = {(uint64_t)a->ldx};
    const uint32_t box[2] = {128, (uint32_t)(swap ? S4_XROWS : M4_BM)};
    int rc = encode_tmap(&p.tmx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  if (wf8) {
    // fp8 weights [E][N][K]: rows past N and values past K read as zero
    const uint64_t dims[3] = {(uint64_t)a->k, (uint64_t)a->n, (uint64_t)a->n_experts};
    const uint64_t strides[2] = {(uint64_t)a->k, (uint64_t)a->k * (uint64_t)a->n};
    const uint32_t box[3] = {128, (uint32_t)M4_BN, 1};
    int rc = encode_tmap(&p.tmw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  } else {
    // blocked weights: one (expert, N tile, K step) block of 256 rows x 64 bytes after the other, so a tile
    // step is one contiguous 16 KB run of HBM
    const uint64_t tiles_n = (uint64_t)((a->n + M4_BN - 1) / M4_BN);
    const uint64_t rows = (uint64_t)a->n_experts * tiles_n * (uint64_t)((a->k + 127) / 128) * M4_BN;
    if (rows > (1ull << 31)) return TB200_ERR_UNSUPPORTED;
    const uint64_t dims[2] = {128, rows};  // in 4-bit values
    const uint64_t strides[1] = {64};
    const uint32_t box[2] = {128, (uint32_t)(swap ? S4_WROWS : M4_BN)};
    int rc = encode_tmap(&p.tmw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, a->w, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.sfw = static_cast<const uint8_t*>(a->w_scale);
  p.slice_offs = a->slice_offs;
  p.slice_sizes = a->slice_sizes;
  p.sched = a->block_schedule;
  p.scatter = a->scatter_indx;
  p.gammas = a->gammas;
  p.bias = a->bias;
  p.x_scale = a->x_scale;
  p.w_flex = a->w_flex_scale;
  p.y_expected = a->y_expected_scale;
  p.y_actual = a->y_actual_scale;
  p.saturate = a->flexpoint_saturate_inf ? 1 : 0;
  p.x_sf = static_cast<const uint8_t*>(a->x_mx_scale);
  p.ld_xsf = a->ld_x_mx_scale;
  p.y_sf = static_cast<uint8_t*>(a->y_mx_scale);
  p.ld_ysf = a->ld_y_mx_scale;
  p.rows_x = (int)a->rows_x;
  p.y = a->y;
  p.ldy = a->ldy;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.n_sched = (int)a->n_sched;
  p.tiles_n = swap ? (int)((a->n + S4_WROWS - 1) / S4_WROWS) : (int)((a->n + M4_BN - 1) / M4_BN);
  if ((long long)p.n_sched * p.tiles_n > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  p.units = p.n_sched * p.tiles_n;
  p.n = (int)a->n;
  p.k_blocks = (int)((a->k + 127) / 128);
  p.n_blocks = (int)((a->n + 127) / 128);
  p.rows_y = (int)a->rows_y;
  p.swiglu = a->swiglu ? 1 : 0;
  p.has_limit = a->swiglu_has_limit ? 1 : 0;
  p.alpha = a->swiglu_alpha;
  p.limit = a->swiglu_limit;
  p.out_kind = a->out_dtype == TB200_F16 ? MOE_OUT_F16 : a->out_dtype == TB200_E4M3 ? MOE_OUT_E4M3
               : a->out_dtype == TB200_E5M2 ? MOE_OUT_E5M2 : MOE_OUT_BF16;
  const uint32_t xfmt = a->x_dtype == TB200_E5M2 ? 1u : 0u;
  const uint32_t wfmt = wf8 ? (a->w_dtype == TB200_E5M2 ? 1u : 0u) : 5u;  // 5 = e2m1
  for (uint32_t k = 0; k < 4; ++k)
    p.idesc[k] = swap ? make_idesc_mx(wfmt, xfmt, S4_WROWS, S4_XROWS, k, k) : make_idesc_mx(xfmt, wfmt, M4_BM, M4_BN, k, k);

  const int grid = p.units < sms ? p.units : sms;
  const bool ext = p.x_sf || p.y_sf || p.w_flex || p.y_expected || p.y_actual;
  if (swap) {
    auto kfn = ext ? moe_gemm_mx4_swap_kernel<true> : moe_gemm_mx4_swap_kernel<false>;
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Mx4SwapSmem::TOTAL) != cudaSuccess)
      return TB200_ERR_CUDA;
    kfn<<<grid, M4_THREADS, Mx4SwapSmem::TOTAL, stream>>>(p);
  } else {
    auto kfn = wf8 ? moe_gemm_mx4_kernel<true, true> : ext ? moe_gemm_mx4_kernel<true, false> : moe_gemm_mx4_kernel<false, false>;
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Mx4Smem::TOTAL) != cudaSuccess)
      return TB200_ERR_CUDA;
    kfn<<<grid, M4_BIG_THREADS, Mx4Smem::TOTAL, stream>>>(p);
  }
  return cuda_err(cudaGetLastError());
}
