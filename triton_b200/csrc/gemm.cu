// Dense GEMM for sm_100a: persistent, warp-specialised, TMA -> shared-memory ring ->
// tcgen05.mma with the accumulator double-buffered in tensor memory -> epilogue warps.
//
// Roles (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer (one
// lane; the warp also owns the TMEM allocation), warps 2..5 = epilogue (each reads its own
// 32-lane quarter of TMEM). Tile = 128 x BN, K step = 128 bytes of K per row (64 16-bit or
// 128 8-bit elements). The same kernel serves bf16/fp16 (kind::f16) and e4m3/e5m2
// (kind::f8f6f4): operand geometry, instruction descriptor and output mode are parameters.
//
// Counterpart in the reference: matmul_kernel_tma_ws_blackwell,
// third_party/tlx/tutorials/blackwell_gemm_ws.py:1168-1483 (producer :961-1088, MMA :840-957,
// epilogue :680-836) and the tensorwise path of blackwell_scaled_mm_ws.py:51-378.
#include "common.cuh"
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
  int is_f8;
  uint32_t idesc;
  OperandGeom ga, gb;
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * STAGE_K_BYTES;
  static constexpr int B_BYTES = BN * STAGE_K_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ void unit_to_tile(const GemmParams& p, int unit, int& pid_m, int& pid_n, int& ks) {
  int tile = unit / p.split_k;
  ks = unit - tile * p.split_k;
  const int group = p.group_m * p.tiles_n;
  const int gid = tile / group;
  const int first_m = gid * p.group_m;
  const int gsz = min(p.tiles_m - first_m, p.group_m);
  const int r = tile - gid * group;
  pid_m = first_m + (r % gsz);
  pid_n = r / gsz;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;

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

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      uint32_t it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x) {
        int pid_m, pid_n, ks;
        unit_to_tile(p, unit, pid_m, pid_n, ks);
        const int m0 = pid_m * BM, n0 = pid_n * BN;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          const int kx = kb * p.bk_elems;
          for (uint32_t i = 0; i < p.ga.boxes; ++i) {
            if (p.ga.mn_major)
              tma_load_2d(sa + i * p.ga.box_bytes, &p.tma, &full[s], m0 + (int)(i * p.ga.box_mn), kx, pol);
            else
              tma_load_2d(sa + i * p.ga.box_bytes, &p.tma, &full[s], kx, m0 + (int)(i * p.ga.box_mn), pol);
          }
          for (uint32_t i = 0; i < p.gb.boxes; ++i) {
            if (p.gb.mn_major)
              tma_load_2d(sb + i * p.gb.box_bytes, &p.tmb, &full[s], n0 + (int)(i * p.gb.box_mn), kx, pol);
            else
              tma_load_2d(sb + i * p.gb.box_bytes, &p.tmb, &full[s], kx, n0 + (int)(i * p.gb.box_mn), pol);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      const uint64_t sw = SWIZZLE_128B;
      for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x, ++tcount) {
        int pid_m, pid_n, ks;
        unit_to_tile(p, unit, pid_m, pid_n, ks);
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        const uint32_t acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1, p.status, WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, p.status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, p.ga.lbo, p.ga.sbo, sw);
          const uint64_t bdesc = make_smem_desc(sb, p.gb.lbo, p.gb.sbo, sw);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = adesc + (uint64_t)((k * p.ga.kstep) >> 4);
            const uint64_t bd = bdesc + (uint64_t)((k * p.gb.kstep) >> 4);
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if (p.is_f8)
              umma_f8_ss(tmem_d, ad, bd, p.idesc, accum);
            else
              umma_f16_ss(tmem_d, ad, bd, p.idesc, accum);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    float alpha = 1.0f;
    if (p.scale_a) alpha *= __ldg(p.scale_a);
    if (p.scale_b) alpha *= __ldg(p.scale_b);
    uint32_t tcount = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < p.units && ok; unit += gridDim.x, ++tcount) {
      int pid_m, pid_n, ks;
      unit_to_tile(p, unit, pid_m, pid_n, ks);
      const int m0 = pid_m * BM, n0 = pid_n * BN;
      const uint32_t acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aph, p.status, WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + c, v);
        tmem_ld_wait();
        const int col = n0 + c;
        if (row < p.m && col < p.n) {
          if (p.out_mode <= 1) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.c) + (long long)row * p.ldc + col;
            const bool vec = (col + 32 <= p.n) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 o;
                uint32_t w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  float lo = __uint_as_float(v[j * 8 + 2 * t]) * alpha;
                  float hi = __uint_as_float(v[j * 8 + 2 * t + 1]) * alpha;
                  w[t] = (p.out_mode == 0) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
                }
                o.x = w[0]; o.y = w[1]; o.z = w[2]; o.w = w[3];
                reinterpret_cast<uint4*>(dst)[j] = o;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.n; ++j) {
                float x = __uint_as_float(v[j]) * alpha;
                if (p.out_mode == 0) {
                  __nv_bfloat16 h = __float2bfloat16_rn(x);
                  dst[j] = *reinterpret_cast<uint16_t*>(&h);
                } else {
                  __half h = __float2half_rn(x);
                  dst[j] = *reinterpret_cast<uint16_t*>(&h);
                }
              }
            }
          } else {
            float* dst = (p.out_mode == 2)
                             ? reinterpret_cast<float*>(p.c) + (long long)row * p.ldc + col
                             : p.ws + ((long long)ks * p.m + row) * (long long)p.n + col;
            const bool vec = (col + 32 <= p.n) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 o;
                o.x = __uint_as_float(v[4 * j]) * alpha;
                o.y = __uint_as_float(v[4 * j + 1]) * alpha;
                o.z = __uint_as_float(v[4 * j + 2]) * alpha;
                o.w = __uint_as_float(v[4 * j + 3]) * alpha;
                reinterpret_cast<float4*>(dst)[j] = o;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.n; ++j) dst[j] = __uint_as_float(v[j]) * alpha;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// C[m,n] = sum_s ws[s,m,n] (fp32) -> out dtype. One thread per 4 consecutive columns.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ c, int m, int n, long long ldc,
                                     int split_k, int out_mode) {
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
  int bn;
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
  if (bn == 0) {
    // Pick the widest tile whose estimated time (waves x per-tile cost) is smallest.
    long long best = -1;
    const int cands[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i) {
      const int cbn = cands[i];
      const long long tiles = tm * ((a->n + cbn - 1) / cbn);
      const long long waves = (tiles + sms - 1) / sms;
      const long long cost = waves * (cbn + 48);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cbn;
      }
    }
  }
  if (bn != 64 && bn != 128 && bn != 256) return false;
  const long long tn = (a->n + bn - 1) / bn;
  const long long tiles = tm * tn;
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
  plan->bn = bn;
  plan->split_k = (int)split;
  plan->kb_per_split = (int)per;
  plan->k_blocks = (int)kb;
  plan->tiles_m = (int)tm;
  plan->tiles_n = (int)tn;
  return true;
}

template <int BN, int STAGES>
static int launch_gemm(const GemmParams& p, int grid, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kfn = gemm_kernel<BN, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
  if (e != cudaSuccess) return TB200_ERR_CUDA;
  kfn<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(p);
  return cuda_err(cudaGetLastError());
}

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

}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_gemm_workspace_bytes(const tb200_gemm_args* a) {
  if (validate(a) != TB200_OK) return 0;
  GemmPlan plan;
  int sms = sm_count();
  if (sms <= 0) sms = 148;
  if (!plan_gemm(a, sms, &plan)) return 0;
  if (plan.split_k <= 1) return 0;
  return (size_t)plan.split_k * (size_t)a->m * (size_t)a->n * sizeof(float);
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
  rc = set_operand(&p.gb, &p.tmb, a->b, a->n, a->k, a->ldb, a->b_k_major, eb, plan.bn, dt);
  if (rc != TB200_OK) return rc;

  uint32_t fmt;
  if (f8)
    fmt = a->in_dtype == TB200_E4M3 ? 0u : 1u;
  else
    fmt = a->in_dtype == TB200_F16 ? 0u : 1u;
  p.idesc = make_idesc(fmt, fmt, p.ga.mn_major, p.gb.mn_major, BM, plan.bn);
  p.is_f8 = f8 ? 1 : 0;
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
  p.status = status_ptr();
  if (!p.status) return TB200_ERR_CUDA;
  const int final_mode = a->out_dtype == TB200_BF16 ? 0 : (a->out_dtype == TB200_F16 ? 1 : 2);
  if (plan.split_k > 1) {
    const size_t need = (size_t)plan.split_k * (size_t)a->m * (size_t)a->n * sizeof(float);
    if (!a->workspace || a->workspace_bytes < need) return TB200_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return TB200_ERR_BAD_ARG;
    p.ws = static_cast<float*>(a->workspace);
    p.out_mode = 3;
  } else {
    p.out_mode = final_mode;
  }
  const int grid = p.units < sms ? p.units : sms;
  switch (plan.bn) {
    case 256: rc = launch_gemm<256, 4>(p, grid, stream); break;
    case 128: rc = launch_gemm<128, 6>(p, grid, stream); break;
    default: rc = launch_gemm<64, 8>(p, grid, stream); break;
  }
  if (rc != TB200_OK) return rc;
  if (plan.split_k > 1) {
    // scale factors were already applied to the partial sums
    const long long total = (long long)a->m * ((a->n + 3) / 4);
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.ws, a->c, p.m, p.n, p.ldc, plan.split_k, final_mode);
    rc = cuda_err(cudaGetLastError());
  }
  return rc;
}
