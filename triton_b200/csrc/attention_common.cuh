// Device helpers shared by the attention forward and backward kernels: fast exp2, packed f32x2
// arithmetic and the per-warpgroup register re-partition.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace tb200 {

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// packed f32x2 arithmetic (two fp32 lanes in one 64-bit register, one issue slot)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 32 columns of this thread's TMEM lane into s[OFF .. OFF+31] (no wait)
// two 16-bit floats (bf16, or fp16 when F16) widened to a packed f32x2
template <bool F16>
__device__ __forceinline__ uint64_t unpack16x2(uint32_t v) {
  if (F16) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    return pack2(f.x, f.y);
  }
  return pack2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

template <int OFF, int N>
__device__ __forceinline__ void tmem_ld_row32(uint32_t taddr, uint32_t (&s)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(s[OFF + 0]), "=r"(s[OFF + 1]), "=r"(s[OFF + 2]), "=r"(s[OFF + 3]), "=r"(s[OFF + 4]), "=r"(s[OFF + 5]),
        "=r"(s[OFF + 6]), "=r"(s[OFF + 7]), "=r"(s[OFF + 8]), "=r"(s[OFF + 9]), "=r"(s[OFF + 10]), "=r"(s[OFF + 11]),
        "=r"(s[OFF + 12]), "=r"(s[OFF + 13]), "=r"(s[OFF + 14]), "=r"(s[OFF + 15]), "=r"(s[OFF + 16]),
        "=r"(s[OFF + 17]), "=r"(s[OFF + 18]), "=r"(s[OFF + 19]), "=r"(s[OFF + 20]), "=r"(s[OFF + 21]),
        "=r"(s[OFF + 22]), "=r"(s[OFF + 23]), "=r"(s[OFF + 24]), "=r"(s[OFF + 25]), "=r"(s[OFF + 26]),
        "=r"(s[OFF + 27]), "=r"(s[OFF + 28]), "=r"(s[OFF + 29]), "=r"(s[OFF + 30]), "=r"(s[OFF + 31])
      : "r"(taddr)
      : "memory");
}

}  // namespace tb200
