// Epilogue pieces shared by the grouped (MoE) GEMM kernels.
#pragma once
#include "common.cuh"

namespace tb200 {

__device__ __forceinline__ float moe_swiglu(float g, float l, float alpha, float limit, int has_limit) {
  if (has_limit) {
    g = fminf(g, limit);
    l = fminf(fmaxf(l, -limit), limit);
  }
  return g / (1.f + __expf(-alpha * g)) * (l + 1.f);
}

// Epilogue of the grouped GEMMs for 32 accumulator columns of one output row: (x acc_scale) + bias ->
// SwiGLU on adjacent (gate, linear) column pairs -> x gamma -> 16-bit store at row out_row.
__device__ __forceinline__ void moe_store_chunk(const uint32_t (&v)[32], uint16_t* y, long long ldy, int out_row, int col,
                                                int n, const float* brow, int swiglu, float alpha, float limit,
                                                int has_limit, float gamma, int out_f16, float acc_scale) {
  float f[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    f[j] = __uint_as_float(v[j]) * acc_scale;
    if (brow && col + j < n) f[j] += __ldg(brow + col + j);
  }
  if (swiglu) {
    // 32 accumulator columns -> 16 outputs at column (col / 2)
    uint16_t* dst = y + (long long)out_row * ldy + (col >> 1);
    const int cnt = min(16, (n - col) >> 1);
    float o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = moe_swiglu(f[2 * j], f[2 * j + 1], alpha, limit, has_limit) * gamma;
    if (cnt == 16 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
          w[t] = out_f16 ? pack_f16x2(o[j * 8 + 2 * t], o[j * 8 + 2 * t + 1])
                         : pack_bf16x2(o[j * 8 + 2 * t], o[j * 8 + 2 * t + 1]);
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < cnt) {
          if (out_f16) {
            __half h = __float2half_rn(o[j]);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          } else {
            __nv_bfloat16 h = __float2bfloat16_rn(o[j]);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          }
        }
      }
    }
  } else {
    uint16_t* dst = y + (long long)out_row * ldy + col;
    const int cnt = min(32, n - col);
    if (cnt == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float lo = f[j * 8 + 2 * t] * gamma, hi = f[j * 8 + 2 * t + 1] * gamma;
          w[t] = out_f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
        }
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < cnt) {
          const float x = f[j] * gamma;
          if (out_f16) {
            __half h = __float2half_rn(x);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          } else {
            __nv_bfloat16 h = __float2bfloat16_rn(x);
            dst[j] = *reinterpret_cast<uint16_t*>(&h);
          }
        }
      }
    }
  }
}

}  // namespace tb200
