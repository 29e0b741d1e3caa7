// bf16 pack / unpack and the activations of the bf16 model kernels.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

namespace cssm {

__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t float2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

// 8 consecutive bf16 (16 bytes) <-> 8 floats
__device__ __forceinline__ void unpack8(const uint4 u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 p = bf16x2_to_float2(w[e]);
    f[2 * e] = p.x; f[2 * e + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = float2_to_bf16x2(f[0], f[1]); u.y = float2_to_bf16x2(f[2], f[3]);
  u.z = float2_to_bf16x2(f[4], f[5]); u.w = float2_to_bf16x2(f[6], f[7]);
  return u;
}

// jax.nn.gelu (tanh form): 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))); tanh.approx is
// within 2^-11 relative, far inside the bf16 model's tolerance.
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

// Two values at a time with packed f32x2 arithmetic (sm_100): half the issue slots of the scalar
// forms in the GEMM epilogues, one MUFU op per value.
__device__ __forceinline__ unsigned long long pk2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(unsigned long long p, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(p));
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ float tanh_approx(float u) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return t;
}
// gelu (tanh form) of a and b in place
__device__ __forceinline__ void gelu_tanh_x2(float& a, float& b) {
  const unsigned long long x = pk2(a, b);
  const unsigned long long x2 = mul2(x, x);
  const unsigned long long inner = fma2(x2, pk2(0.044715f * 0.7978845608028654f, 0.044715f * 0.7978845608028654f),
                                        pk2(0.7978845608028654f, 0.7978845608028654f));
  float ua, ub;
  upk2(mul2(inner, x), ua, ub);
  const unsigned long long hx = mul2(x, pk2(0.5f, 0.5f));
  upk2(fma2(hx, pk2(tanh_approx(ua), tanh_approx(ub)), hx), a, b);
}
// silu(x) = x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)) of a and b in place
__device__ __forceinline__ void silu_tanh_x2(float& a, float& b) {
  const unsigned long long hx = mul2(pk2(a, b), pk2(0.5f, 0.5f));
  float ha, hb;
  upk2(hx, ha, hb);
  upk2(fma2(hx, pk2(tanh_approx(ha), tanh_approx(hb)), hx), a, b);
}

}  // namespace cssm
