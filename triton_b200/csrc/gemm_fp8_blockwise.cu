// Block-wise scaled FP8 GEMM for sm_100a (the "DeepSeek" scheme):
//   C[m, n] = sum_g  (sum_{k in group g} A[m, k] B[n, k]) * scale_a[m, g] * scale_b[n / 128, g]
// with K groups of 128, A [M, K] and B [N, K] fp8 (e4m3 / e5m2) row-major, scale_a stored M-major
// ([K/128][M] in memory), scale_b [N/128][K/128] row-major.
//
// The scales change every 128 values of K, so the sum over K cannot stay in one tensor-memory
// accumulator: each K group is multiplied into a fresh 128 x 256 fp32 partial in TMEM (two partial
// buffers = all 512 columns) and "promoted" - scaled and added to a running sum held in registers.
// Roles (320 threads), one 128 x 256 output tile at a time, persistent over tiles:
//   warp 0        TMA: A (128 x 128 bytes) and B (256 x 128 bytes) of one K group per stage, 4 stages.
//   warp 1        one thread issues four kind::f8f6f4 MMAs (K = 32 each) per K group, the first one
//                 overwriting the partial; it probes the next stage's barrier ahead of them.
//   warps 2-5     promotion group 0: output columns 0-127;  warps 6-9: columns 128-255. Thread t owns
//                 output row t: 128 fp32 running sums in registers; per K group it reads its row of the
//                 partial (tcgen05.ld), multiplies by scale_a[row, g] * scale_b[block, g] (loaded ahead
//                 of the wait) and accumulates; the last group is followed by the conversion and store.
// The partial buffers are released per K group, so the MMAs of the next tile run under the stores.
//
// Counterpart in the reference: _scaled_mm_ws with SCALE_MODE == 0 (blockwise),
// third_party/tlx/tutorials/blackwell_scaled_mm_ws.py:195-217 (scale loads), :300-341 (promotion),
// host entry blackwell_scaled_mm_ws :392; check expression testing/test_correctness.py:535-547.
#include <string.h>

#include "gemm_common.cuh"
#include "host_common.h"

namespace tb200 {

static constexpr int BW_THREADS = 320;
static constexpr int BW_BM = 128;
static constexpr int BW_BN = 256;
static constexpr int BW_KG = 128;  // K group = one pipeline stage = 128 bytes per row
static constexpr int BW_STAGES = 4;

struct BwParams {
  CUtensorMap tma, tmb;  // 2-D (K, rows) fp8, box (128, 128) / (128, 256), 128-byte swizzle
  void* c;
  const float* sa;  // [K/128][M]
  const float* sb;  // [N/128][K/128]
  int* status;
  int m, n;
  long long ldc;
  int k_groups, tiles_m, tiles_n, units, group_m;
  int out_mode;  // 0 bf16, 1 fp16, 2 fp32
  uint32_t idesc;
};

struct BwSmem {
  static constexpr int A_BYTES = BW_BM * BW_KG;
  static constexpr int B_BYTES = BW_BN * BW_KG;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KB
  static constexpr int BAR_OFFSET = BW_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * BW_STAGES + 4) * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(BW_THREADS, 1) gemm_fp8_blockwise_kernel(const __grid_constant__ BwParams p) {
  using L = BwSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + BW_STAGES;
  uint64_t* pfull = empty + BW_STAGES;  // [2] MMA -> promotion: partial of one K group complete
  uint64_t* pempty = pfull + 2;         // [2] promotion -> MMA: partial read out (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + 2);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.tma);
    tma_prefetch_desc(&p.tmb);
    for (int s = 0; s < BW_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&pfull[i], 1);
      mbar_init(&pempty[i], 256);
    }
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
  int* const status = p.status;
  const int units = p.units, k_groups = p.k_groups;
  const uint32_t smem_a = smem_u32(smem);
  const uint32_t full_a = smem_u32(full), empty_a = smem_u32(empty);
  const uint32_t pfull_a = smem_u32(pfull), pempty_a = smem_u32(pempty);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        const TileCoord t = unit_to_tile(unit, 1, p.group_m, p.tiles_m, p.tiles_n);
        const int m0 = t.pid_m * BW_BM, n0 = t.pid_n * BW_BN;
        for (int g = 0; g < k_groups; ++g) {
          if (!mbar_wait_a(empty_a + s * 8, ph ^ 1, status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t bar = full_a + s * 8;
          mbar_expect_tx_a(bar, L::STAGE_BYTES);
          const uint32_t sa = smem_a + s * L::STAGE_BYTES;
          tma_load_2d_a(sa, &p.tma, bar, g * BW_KG, m0, pol);
          tma_load_2d_a(sa + L::A_BYTES, &p.tmb, bar, g * BW_KG, n0, pol);
          if (++s == BW_STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = p.idesc;
      const uint64_t adesc0 = make_smem_desc(smem_a, 16, 1024, SWIZZLE_128B);
      const uint64_t bdesc0 = make_smem_desc(smem_a + L::A_BYTES, 16, 1024, SWIZZLE_128B);
      uint32_t s = 0, ph = 0, cnt = 0;
      bool ok = true, ready = false;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        for (int g = 0; g < k_groups; ++g, ++cnt) {
          const uint32_t buf = cnt & 1;
          if (!mbar_wait_a(pempty_a + buf * 8, ((cnt >> 1) & 1) ^ 1, status, WAIT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (!ready && !mbar_wait_a(full_a + s * 8, ph, status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s1 = (s + 1 == BW_STAGES) ? 0 : s + 1;
          ready = mbar_test_a(full_a + s1 * 8, s1 == 0 ? ph ^ 1 : ph);  // probe ahead of the MMAs
          const uint32_t tmem_d = tmem_base + buf * BW_BN;
          const uint64_t ad = adesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(s * (L::STAGE_BYTES >> 4));
          umma_f8_ss(tmem_d, ad, bd, idesc, 0u);
          umma_f8_ss(tmem_d, ad + 2, bd + 2, idesc, 1u);
          umma_f8_ss(tmem_d, ad + 4, bd + 4, idesc, 1u);
          umma_f8_ss(tmem_d, ad + 6, bd + 6, idesc, 1u);
          umma_commit_a(empty_a + s * 8);
          umma_commit_a(pfull_a + buf * 8);
          s = s1;
          if (s == 0) ph ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------- promotion + epilogue
    const int w = (warp - 2) >> 2;  // column half of the tile
    const int q = warp & 3;         // TMEM lane quadrant of this warp
    const int r = q * 32 + lane;
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + w * 128;
    const float* const sa = p.sa;
    const float* const sb = p.sb;
    const int m = p.m, n = p.n;
    uint32_t cnt = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      const TileCoord t = unit_to_tile(unit, 1, p.group_m, p.tiles_m, p.tiles_n);
      const int row = t.pid_m * BW_BM + r;
      const int col0 = t.pid_n * BW_BN + w * 128;
      const bool row_ok = row < m, col_ok = col0 < n;  // N is a multiple of 128: a half is all in or all out
      const float* sb_row = sb + (size_t)(col_ok ? col0 / 128 : 0) * k_groups;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      float scale = (row_ok ? __ldg(sa + row) : 0.f) * __ldg(sb_row);
      for (int g = 0; g < k_groups; ++g, ++cnt) {
        const uint32_t buf = cnt & 1;
        // the next group's factor is loaded before this group's wait
        float scale_next = 0.f;
        if (g + 1 < k_groups) scale_next = (row_ok ? __ldg(sa + (size_t)(g + 1) * m + row) : 0.f) * __ldg(sb_row + g + 1);
        if (!mbar_wait_a(pfull_a + buf * 8, (cnt >> 1) & 1, status, WAIT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + buf * BW_BN + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(v[i]), scale, acc[c * 32 + i]);
        }
        tc_fence_before_sync();
        mbar_arrive_a(pempty_a + buf * 8);
        scale = scale_next;
      }
      if (!ok) break;
      if (col_ok) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(acc[c * 32 + i]);
          store_chunk(p.c, nullptr, p.ldc, m, n, p.out_mode, v, row, col0 + c * 32, 0, 1.f);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_gemm_fp8_blockwise(const tb200_gemm_fp8_blockwise_args* a, void* stream_) {
  if (!a || !a->a || !a->b || !a->c || !a->scale_a || !a->scale_b) return TB200_ERR_BAD_ARG;
  if (a->m < 0 || a->n < 0 || a->k < 0) return TB200_ERR_BAD_ARG;
  if (a->in_dtype != TB200_E4M3 && a->in_dtype != TB200_E5M2) return TB200_ERR_UNSUPPORTED;
  if (a->out_dtype != TB200_BF16 && a->out_dtype != TB200_F16 && a->out_dtype != TB200_F32) return TB200_ERR_UNSUPPORTED;
  if (a->k % BW_KG != 0 || a->n % 128 != 0 || a->k == 0) return TB200_ERR_BAD_ARG;
  if (a->m == 0 || a->n == 0) return TB200_OK;
  if (a->m > INT32_MAX || a->n > INT32_MAX || a->k > INT32_MAX || a->ldc < a->n) return TB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15)) return TB200_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int sms = sm_count();
  if (sms <= 0) return TB200_ERR_CUDA;

  BwParams p;
  memset(&p, 0, sizeof(p));
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->m};
    const uint64_t strides[1] = {(uint64_t)a->k};
    const uint32_t box[2] = {BW_KG, BW_BM};
    int rc = encode_tmap(&p.tma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->n};
    const uint64_t strides[1] = {(uint64_t)a->k};
    const uint32_t box[2] = {BW_KG, BW_BN};
    int rc = encode_tmap(&p.tmb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
  }
  p.c = a->c;
  p.sa = a->scale_a;
  p.sb = a->scale_b;
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  p.m = (int)a->m;
  p.n = (int)a->n;
  p.ldc = a->ldc;
  p.k_groups = (int)(a->k / BW_KG);
  p.tiles_m = (int)((a->m + BW_BM - 1) / BW_BM);
  p.tiles_n = (int)((a->n + BW_BN - 1) / BW_BN);
  if ((long long)p.tiles_m * p.tiles_n > INT32_MAX) return TB200_ERR_UNSUPPORTED;
  p.units = p.tiles_m * p.tiles_n;
  p.group_m = 8;
  p.out_mode = a->out_dtype == TB200_BF16 ? 0 : (a->out_dtype == TB200_F16 ? 1 : 2);
  const uint32_t fmt = a->in_dtype == TB200_E5M2 ? 1u : 0u;
  p.idesc = make_idesc(fmt, fmt, 0u, 0u, BW_BM, BW_BN);

  auto kfn = gemm_fp8_blockwise_kernel;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, BwSmem::TOTAL) != cudaSuccess)
    return TB200_ERR_CUDA;
  const int grid = p.units < sms ? p.units : sms;
  kfn<<<grid, BW_THREADS, BwSmem::TOTAL, stream>>>(p);
  return cuda_err(cudaGetLastError());
}
