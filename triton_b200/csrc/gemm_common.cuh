// Pieces shared by the GEMM kernels: tile scheduling order and the epilogue's row-chunk store.
#pragma once
#include "common.cuh"

namespace tb200 {

struct TileCoord {
  int pid_m, pid_n, ks;
};

__device__ __forceinline__ TileCoord unit_to_tile(int unit, int split_k, int group_m, int tiles_m, int tiles_n) {
  TileCoord t;
  const int tile = unit / split_k;
  t.ks = unit - tile * split_k;
  const int group = group_m * tiles_n;
  const int gid = tile / group;
  const int first_m = gid * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = tile - gid * group;
  t.pid_m = first_m + (r % gsz);
  t.pid_n = r / gsz;
  return t;
}

// One 32-byte global store (sm_100: 256-bit vector stores); dst 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e,
                                             uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d),
               "r"(e), "r"(f), "r"(g), "r"(h)
               : "memory");
}

// Converts 32 consecutive columns of the thread's row (fp32 accumulators in v) to the 16-bit output type and puts
// them into a 32-row x 128-byte staging buffer in the 128-byte-swizzle order a TMA store expects: row = lane, the
// 16-byte chunk j of the row at ((j ^ (row & 7)) << 4). chunk0 = 0 for the first 32 columns of the 64, 4 for the rest.
__device__ __forceinline__ void stage_chunk(uint32_t buf, int lane, int chunk0, const uint32_t (&v)[32], int col,
                                            int out_mode, float alpha, const float* col_scale, int n) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float lo = __uint_as_float(v[j * 8 + 2 * t]) * alpha;
      float hi = __uint_as_float(v[j * 8 + 2 * t + 1]) * alpha;
      if (col_scale) {  // columns past n are clipped by the store; their factors are not read
        const int cidx = col + j * 8 + 2 * t;
        lo *= cidx < n ? __ldg(col_scale + cidx) : 0.f;
        hi *= cidx + 1 < n ? __ldg(col_scale + cidx + 1) : 0.f;
      }
      w[t] = (out_mode == 0) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
    }
    const uint32_t addr = buf + (uint32_t)lane * 128 + ((uint32_t)((chunk0 + j) ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
  }
}

// Writes 32 consecutive columns of one output row (fp32 accumulators in v) in the output mode.
__device__ __forceinline__ void store_chunk(void* c, float* ws, long long ldc, int m, int n, int out_mode,
                                            uint32_t (&v)[32], int row, int col, int ks, float alpha,
                                            const float* col_scale = nullptr) {
  if (row >= m || col >= n) return;
  const bool full = col + 32 <= n;
  if (col_scale) {  // per-column factors (row-wise scaled GEMM); alpha then carries the row's factor
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (full || col + j < n) v[j] = __float_as_uint(__uint_as_float(v[j]) * __ldg(col_scale + col + j));
  }
  if (out_mode <= 1) {
    uint16_t* dst = reinterpret_cast<uint16_t*>(c) + (long long)row * ldc + col;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 31) == 0)) {
      // two 32-byte stores: each instruction writes whole sectors (a thread owns a row, so 16-byte stores
      // leave every sector half written per instruction, which the write path handles at half the rate)
      uint32_t w[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float lo = __uint_as_float(v[2 * t]) * alpha;
        const float hi = __uint_as_float(v[2 * t + 1]) * alpha;
        w[t] = (out_mode == 0) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
      }
      st_global_v8(dst, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
      st_global_v8(dst + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
    } else if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float lo = __uint_as_float(v[j * 8 + 2 * t]) * alpha;
          const float hi = __uint_as_float(v[j * 8 + 2 * t + 1]) * alpha;
          w[t] = (out_mode == 0) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
        }
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      const int cnt = n - col;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < cnt) {
          const float x = __uint_as_float(v[j]) * alpha;
          if (out_mode == 0) {
            __nv_bfloat16 h = __float2bfloat16_rn(x);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          } else {
            __half h = __float2half_rn(x);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          }
        }
      }
    }
  } else {
    float* dst = (out_mode == 2) ? reinterpret_cast<float*>(c) + (long long)row * ldc + col
                                 : ws + ((long long)ks * m + row) * (long long)n + col;
    if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        reinterpret_cast<float4*>(dst)[j] =
            make_float4(__uint_as_float(v[4 * j]) * alpha, __uint_as_float(v[4 * j + 1]) * alpha,
                        __uint_as_float(v[4 * j + 2]) * alpha, __uint_as_float(v[4 * j + 3]) * alpha);
      }
    } else {
      const int cnt = n - col;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < cnt) dst[j] = __uint_as_float(v[j]) * alpha;
    }
  }
}


}  // namespace tb200
