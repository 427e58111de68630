// Epilogue pieces shared by the grouped (MoE) GEMM kernels.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace tb200 {

__device__ __forceinline__ float moe_swiglu(float g, float l, float alpha, float limit, int has_limit) {
  if (has_limit) {
    g = fminf(g, limit);
    l = fminf(fmaxf(l, -limit), limit);
  }
  return g / (1.f + __expf(-alpha * g)) * (l + 1.f);
}

// Output element kinds of the grouped GEMMs' epilogue.
enum MoeOutKind : int { MOE_OUT_BF16 = 0, MOE_OUT_F16 = 1, MOE_OUT_E4M3 = 2, MOE_OUT_E5M2 = 3 };

__device__ __forceinline__ uint32_t moe_pack16(float lo, float hi, int kind) {
  return kind == MOE_OUT_F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}

// Two floats -> two fp8 bytes (low byte = lo), round to nearest even, saturating to the largest finite value:
// the conversion the reference's kernels perform when the output tensor is fp8 (cvt.rn.satfinite).
__device__ __forceinline__ uint32_t moe_pack8(float lo, float hi, int kind) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE,
                                            kind == MOE_OUT_E5M2 ? __NV_E5M2 : __NV_E4M3);
}

__device__ __forceinline__ void moe_store_one(void* y, long long elem, float x, int kind) {
  if (kind >= MOE_OUT_E4M3) {
    static_cast<uint8_t*>(y)[elem] = (uint8_t)(moe_pack8(x, 0.f, kind) & 0xffu);
  } else {
    static_cast<uint16_t*>(y)[elem] = (uint16_t)(moe_pack16(x, 0.f, kind) & 0xffffu);
  }
}

// N (16 or 32) consecutive outputs of one row starting at element `elem`; the first `cnt` exist. 16-byte stores
// when the run is whole and aligned, element stores otherwise.
template <int N>
__device__ __forceinline__ void moe_store_run(void* y, long long elem, const float (&o)[N], int cnt, int kind) {
  if (kind >= MOE_OUT_E4M3) {
    uint8_t* dst = static_cast<uint8_t*>(y) + elem;
    if (cnt == N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < N / 16; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
          w[t] = moe_pack8(o[j * 16 + 4 * t], o[j * 16 + 4 * t + 1], kind) |
                 (moe_pack8(o[j * 16 + 4 * t + 2], o[j * 16 + 4 * t + 3], kind) << 16);
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
  } else {
    uint16_t* dst = static_cast<uint16_t*>(y) + elem;
    if (cnt == N && ((reinterpret_cast<uintptr_t>(dst) & 31) == 0)) {
      // 32-byte stores: a thread owns a row, so each instruction then writes whole sectors
#pragma unroll
      for (int j = 0; j < N / 16; ++j) {
        uint32_t w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = moe_pack16(o[j * 16 + 2 * t], o[j * 16 + 2 * t + 1], kind);
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + j * 16), "r"(w[0]), "r"(w[1]),
                     "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
      }
      return;
    }
    if (cnt == N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < N / 8; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) w[t] = moe_pack16(o[j * 8 + 2 * t], o[j * 8 + 2 * t + 1], kind);
        reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j)
    if (j < cnt) moe_store_one(y, elem + j, o[j], kind);
}

// Optional terms of the epilogue beyond bias / activation / gamma (matmul.py:245-256 in the reference): a per-row
// factor on the bias (betas), one factor on the biased accumulator (out_alpha), and a 16-bit matrix added to the
// result (c_acc_in; may be the output itself).
struct MoeEpilogueExtra {
  float beta = 1.f;          // betas[sorted row]
  float out_alpha = 1.f;
  const void* acc_in = nullptr;  // row-major 16-bit matrix, same kind as the output
  long long ld_acc = 0;
  // flexpoint output (numerics_details/flexpoint.py:155-188 float_to_flex): the largest |output| is reported
  // (track_absmax; the caller folds it into actual_scale), then the output is multiplied by 1 / expected_scale
  // and, on request, clamped to the finite range of the output type
  float inv_expected = 1.f;
  float clip = 0.f;  // > 0: clamp to [-clip, clip]
  int track_absmax = 0;
};

// actual_scale of a flexpoint output from the largest |output|: absmax * (1 / max_finite) + 1e-30 with the
// reference's rounded-up reciprocal constants (flexpoint.py:17-21,133-142); NaN counts as +inf.
__device__ __forceinline__ float moe_flex_scale(float absmax, int kind) {
  const uint32_t bits = min(__float_as_uint(absmax) & 0x7FFFFFFFu, 0x7F800000u);
  const uint32_t rcp = kind == MOE_OUT_E5M2 ? 0x37924925u : kind == MOE_OUT_F16 ? 0x37802008u : 0x3B124925u;
  return fmaf(__uint_as_float(bits), __uint_as_float(rcp), 1.0e-30f);
}

// one warp's contribution to actual_scale (positive floats order like their bit patterns)
__device__ __forceinline__ void moe_flex_publish(float absmax, float* actual_scale, int kind) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, d));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(actual_scale), __float_as_int(moe_flex_scale(absmax, kind)));
}

// o[j] += acc_in[elem + j] for the first cnt values (16-bit matrix of the output's kind)
template <int N>
__device__ __forceinline__ void moe_add_acc(float (&o)[N], int cnt, const void* acc_in, long long elem, int kind) {
  const uint16_t* src = static_cast<const uint16_t*>(acc_in) + elem;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    if (j < cnt) {
      const uint16_t raw = src[j];
      o[j] += kind == MOE_OUT_F16 ? __half2float(*reinterpret_cast<const __half*>(&raw)) : __uint_as_float((uint32_t)raw << 16);
    }
  }
}

// Epilogue of the grouped GEMMs for 32 accumulator columns of one output row, in the reference's order
// (_p_matmul.py:606-622): (x acc_scale) + bias * beta -> x out_alpha -> SwiGLU on adjacent (gate, linear) column
// pairs -> x gamma -> + acc_in -> (flexpoint: absmax, x 1 / expected_scale, clamp) -> store at row out_row (ldy in
// elements). Returns the largest |output| before the flexpoint scaling (0 unless asked for).
__device__ __forceinline__ float moe_store_chunk(const uint32_t (&v)[32], void* y, long long ldy, int out_row, int col,
                                                 int n, const float* brow, int swiglu, float alpha, float limit,
                                                 int has_limit, float gamma, int out_kind, float acc_scale,
                                                 const MoeEpilogueExtra ex = MoeEpilogueExtra()) {
  float f[32];
  float absmax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    f[j] = __uint_as_float(v[j]) * acc_scale;
    if (brow && col + j < n) f[j] += __ldg(brow + col + j) * ex.beta;
    f[j] *= ex.out_alpha;
  }
  if (swiglu) {
    // 32 accumulator columns -> 16 outputs at column (col / 2)
    float o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = moe_swiglu(f[2 * j], f[2 * j + 1], alpha, limit, has_limit) * gamma;
    const int cnt = min(16, (n - col) >> 1);
    if (ex.acc_in) moe_add_acc<16>(o, cnt, ex.acc_in, (long long)out_row * ex.ld_acc + (col >> 1), out_kind);
    if (ex.track_absmax || ex.inv_expected != 1.f || ex.clip > 0.f) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (j < cnt) absmax = fmaxf(absmax, fabsf(o[j]));
        o[j] *= ex.inv_expected;
        if (ex.clip > 0.f) o[j] = fminf(fmaxf(o[j], -ex.clip), ex.clip);
      }
    }
    moe_store_run<16>(y, (long long)out_row * ldy + (col >> 1), o, cnt, out_kind);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] *= gamma;
    const int cnt = min(32, n - col);
    if (ex.acc_in) moe_add_acc<32>(f, cnt, ex.acc_in, (long long)out_row * ex.ld_acc + col, out_kind);
    if (ex.track_absmax || ex.inv_expected != 1.f || ex.clip > 0.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < cnt) absmax = fmaxf(absmax, fabsf(f[j]));
        f[j] *= ex.inv_expected;
        if (ex.clip > 0.f) f[j] = fminf(fmaxf(f[j], -ex.clip), ex.clip);
      }
    }
    moe_store_run<32>(y, (long long)out_row * ldy + col, f, cnt, out_kind);
  }
  return absmax;
}

// The same epilogue up to the store: the outputs of a 32-column accumulator chunk written to o[OFF ..] - 32 values
// (OFF = 0), or 16 with SwiGLU (OFF = 0 or 16, so that two chunks fill one block of 32 outputs).
template <int OFF>
__device__ __forceinline__ void moe_chunk_values(const uint32_t (&v)[32], int col, int n, const float* brow, int swiglu,
                                                 float alpha, float limit, int has_limit, float gamma, float acc_scale,
                                                 const MoeEpilogueExtra ex, float (&o)[32]) {
  float f[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    f[j] = __uint_as_float(v[j]) * acc_scale;
    if (brow && col + j < n) f[j] += __ldg(brow + col + j) * ex.beta;
    f[j] *= ex.out_alpha;
  }
  if (swiglu) {
#pragma unroll
    for (int j = 0; j < 16; ++j) o[OFF + j] = moe_swiglu(f[2 * j], f[2 * j + 1], alpha, limit, has_limit) * gamma;
  } else if (OFF == 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = f[j] * gamma;
  }
}

// One MX block of the output: 32 consecutive values of a row (the first cnt exist) share an e8m0 scale
// 2^ceil(log2(amax / max_finite)) - in bits (bits(amax / max_finite) + 0x7FFFFF) & 0x7F800000 -, each value is
// multiplied by the reciprocal of that scale (by 0 when the scale is 0) and converted to fp8 with round to nearest
// even. This is the reference's quantize_mxfp8_fn epilogue (numerics_details/mxfp_details/_downcast_to_mxfp.py:
// 34-85, rounding mode ROUND_UP) and its torch twin downcast_to_mxfp_torch. dst: the block's first output byte;
// scale_dst: its scale byte.
__device__ __forceinline__ void moe_store_mx_block(const float (&o)[32], int cnt, void* y, long long elem,
                                                   uint8_t* scale_dst, int kind) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < cnt) amax = fmaxf(amax, fabsf(o[j]));
  const float max_finite = kind == MOE_OUT_E5M2 ? 57344.f : 448.f;
  const uint32_t bits = (__float_as_uint(__fdiv_rn(amax, max_finite)) + 0x007FFFFFu) & 0x7F800000u;
  const float inv = bits == 0u ? 0.f : __frcp_rn(__uint_as_float(bits));
  *scale_dst = (uint8_t)(bits >> 23);
  float q[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) q[j] = j < cnt ? o[j] * inv : 0.f;
  moe_store_run<32>(y, elem, q, cnt, kind);
}

}  // namespace tb200
