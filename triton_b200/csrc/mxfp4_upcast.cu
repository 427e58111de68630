// MXFP4 weight -> bf16 / fp16 upcast, from the blocked layout tb200_moe_gemm_mx4 reads into the K-contiguous
// [E][N][K] matrix tb200_moe_gemm takes with w_n_major = 0.
//
// Why it exists: with 16-bit activations the reference multiplies an MXFP4 weight by upcasting it to bf16 inside
// its kernel and running the ordinary 16-bit MMA (python/triton_kernels/triton_kernels/matmul_details/_matmul.py:
// 485-489: tl.dot_scaled(x, None, "bf16", w, w_scales, "e2m1")); value * 2^(scale - 127) is exact in bf16, so
// the product equals a bf16 GEMM over the upcast weight. Here the upcast is its own pass - HBM-bound, 0.53
// bytes read and 2 written per weight - and the GEMM is the existing 16-bit grouped kernel.
//
// A CTA walks 256-row x 64-byte blocks of the weight. A thread takes one 4-byte word (8 codes -> one 16-byte
// store) of 16 rows; the 16 lanes of a half-warp cover a row's 64-byte K run, so every load instruction of a
// warp reads 128 contiguous bytes and every store writes two whole 256-byte runs (full sectors: with a thread
// per 16-byte quarter and four stores each, every store instruction wrote half sectors - 3.2 TB/s).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/triton_b200.h"
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int UP_THREADS = 256;

// Two e2m1 codes (one byte, low nibble first) -> two 16-bit floats in one word, without a table: a code's three
// magnitude bits e1 e0 m, placed so that e lands in the two lowest exponent bits and m in the highest mantissa bit,
// ARE the code's value times 2^-B in the target format, the subnormal code 0.5 included (B = 126 for bf16, 14 for
// fp16). MANT is the mantissa width (7 / 10).
template <int MANT>
__device__ __forceinline__ uint32_t e2m1x2_bits(uint32_t byte) {
  const uint32_t t = (byte & 0x0fu) | ((byte & 0xf0u) << 12);  // codes at bits 3:0 and 19:16
  return ((t & 0x00070007u) << (MANT - 1)) | ((t & 0x00080008u) << 12);
}

template <typename T>
struct Upcast;

// bf16: bits * 2^126 is the code's value; times the scale as bf16 (exponent byte = the e8m0 byte: 0 -> 0.0 and
// 255 -> infinity, the very floats the reference's torch upcast multiplies by, numerics_details/mxfp.py
// upcast_from_mxfp_torch). Both products are exact or round once (subnormal results); the NaN-keeping min / max
// then clamp infinities to the largest finite value, as the reference's clamp does.
template <>
struct Upcast<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t scale_word(uint32_t sb) { return (sb << 7) * 0x00010001u; }
  static __device__ __forceinline__ uint32_t run(uint32_t byte, uint32_t scale2) {
    const uint32_t raw = e2m1x2_bits<7>(byte);
    const uint32_t k126 = 0x7e807e80u, big = 0x7f7f7f7fu, nbig = 0xff7fff7fu;
    __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&raw),
                               *reinterpret_cast<const __nv_bfloat162*>(&k126));
    v = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
    v = __hmax2_nan(__hmin2_nan(v, *reinterpret_cast<const __nv_bfloat162*>(&big)),
                    *reinterpret_cast<const __nv_bfloat162*>(&nbig));
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// fp16: the scale's range is far wider than the format's, so the product is formed in fp32 (bits * 2^14 is the
// code's value), clamped to +-65504 with NaN kept, and rounded once.
template <>
struct Upcast<__half> {
  static __device__ __forceinline__ uint32_t scale_word(uint32_t sb) { return sb << 23; }
  static __device__ __forceinline__ uint32_t run(uint32_t byte, uint32_t scale_bits) {
    const uint32_t raw = e2m1x2_bits<10>(byte);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
    const float sc = __uint_as_float(scale_bits);
    float lo = f.x * 16384.f * sc, hi = f.y * 16384.f * sc;
    lo = (lo != lo) ? lo : fminf(fmaxf(lo, -65504.f), 65504.f);
    hi = (hi != hi) ? hi : fminf(fmaxf(hi, -65504.f), 65504.f);
    __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
};

template <typename T>
__global__ void __launch_bounds__(UP_THREADS) mxfp4_upcast_kernel(const uint32_t* __restrict__ w,
                                                                   const uint8_t* __restrict__ w_scale,
                                                                   T* __restrict__ out, int64_t k, int64_t n,
                                                                   int64_t blocks) {
  const int64_t kb_count = k / 128;
  const int64_t n_tiles = (n + 255) / 256;
  const int c = threadIdx.x & 15;   // 4-byte word of the row's 64-byte K run: values 8 c .. 8 c + 7
  const int rb = threadIdx.x >> 4;  // rows rb, rb + 16, ...
  for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
    // b over [E][n_tiles][kb]: one 256-row x 64-byte block of the weight
    const int64_t kb = b % kb_count;
    const int64_t t = (b / kb_count) % n_tiles;
    const int64_t e = b / (kb_count * n_tiles);
    const uint32_t* src = w + b * 4096 + c;
    const int rows = (int)((n - t * 256 < 256) ? n - t * 256 : 256);
    // scale atoms: [n/128][kb][n%32][n/32%4][k/32%4]; row r of this block: atom (2 t + r / 128), the rest from r
    const uint8_t* sc0 = w_scale + ((e * (n / 128) + 2 * t) * kb_count + kb) * 512 + (c >> 2);
    T* dst0 = out + (e * n + t * 256) * k + kb * 128 + c * 8;
    uint32_t codes[16];
    uint32_t sb[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = rb + 16 * i;
      if (r < rows) {
        codes[i] = __ldg(src + r * 16);
        sb[i] = __ldg(sc0 + (int64_t)(r >> 7) * kb_count * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4);
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = rb + 16 * i;
      if (r < rows) {
        const uint32_t sw = Upcast<T>::scale_word(sb[i]);
        uint4 o;
        o.x = Upcast<T>::run(codes[i] & 0xffu, sw);
        o.y = Upcast<T>::run((codes[i] >> 8) & 0xffu, sw);
        o.z = Upcast<T>::run((codes[i] >> 16) & 0xffu, sw);
        o.w = Upcast<T>::run(codes[i] >> 24, sw);
        *reinterpret_cast<uint4*>(dst0 + (int64_t)r * k) = o;
      }
    }
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_mxfp4_upcast(const tb200_mxfp4_upcast_args* a, void* stream_) {
  using namespace tb200;
  if (!a || !a->w || !a->w_scale || !a->out) return TB200_ERR_BAD_ARG;
  if (a->n_experts < 0 || a->k < 0 || a->n < 0) return TB200_ERR_BAD_ARG;
  if (a->k % 128 || a->n % 128) return TB200_ERR_UNSUPPORTED;
  if (a->out_dtype != TB200_BF16 && a->out_dtype != TB200_F16) return TB200_ERR_UNSUPPORTED;
  if (((uintptr_t)a->w | (uintptr_t)a->out) & 15) return TB200_ERR_BAD_ARG;
  const int64_t blocks = a->n_experts * ((a->n + 255) / 256) * (a->k / 128);
  if (blocks == 0) return TB200_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess) return TB200_ERR_CUDA;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap = (int64_t)sms * 8;  // 8 resident CTAs per SM; each walks the blocks with a grid stride
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (a->out_dtype == TB200_BF16)
    mxfp4_upcast_kernel<__nv_bfloat16><<<grid, UP_THREADS, 0, stream>>>(
        (const uint32_t*)a->w, (const uint8_t*)a->w_scale, (__nv_bfloat16*)a->out, a->k, a->n, blocks);
  else
    mxfp4_upcast_kernel<__half><<<grid, UP_THREADS, 0, stream>>>((const uint32_t*)a->w, (const uint8_t*)a->w_scale,
                                                                 (__half*)a->out, a->k, a->n, blocks);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_CUDA;
}
