// Small arithmetic helpers shared by the attention kernels: exp2 on the special-function unit and on the FMA pipe,
// three-input maximum, and the packed two-lane fp32 operations of sm_100.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace attn_util {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^a for a <= 0 on the FMA pipe (the special-function unit, 4 lanes per scheduler, is the bottleneck of the softmax:
// a share of the exponentials goes here instead): round a to an integer n with the 1.5 * 2^23 trick, a cubic for
// 2^(a - n) on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding of P), and n added into the exponent.
__device__ __forceinline__ float ex2_fma(float a) {
  a = fmaxf(a, -120.f);
  const float t = a + 12582912.f;
  const float f = a - (t - 12582912.f);
  float q = fmaf(0.05517157167196274f, f, 0.2426111102104187f);
  q = fmaf(q, f, 0.6932610273361206f);
  q = fmaf(q, f, 0.9999280571937561f);
  return __uint_as_float(__float_as_uint(q) + (__float_as_uint(t) << 23));
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// two fp32 lanes per instruction
__device__ __forceinline__ unsigned long long pack2(uint32_t lo, uint32_t hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

}  // namespace attn_util
