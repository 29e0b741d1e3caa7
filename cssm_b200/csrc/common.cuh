// Shared helpers for the cssm_b200 CUDA sources (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/cssm_b200.h"

#ifndef CSSM_F32X2
#define CSSM_F32X2 1
#endif

namespace cssm {

struct __align__(8) cf {
  float x, y;
};

__device__ __forceinline__ cf mk(float x, float y) { cf r; r.x = x; r.y = y; return r; }
// Complex add / subtract as one packed fp32x2 instruction (sm_100): halves the issue slots of
// the FFT butterflies, which are mostly complex additions.
__device__ __forceinline__ cf operator+(cf a, cf b) {
#if CSSM_F32X2
  unsigned long long pa, pb, pr;
  asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(pb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(pr) : "l"(pa), "l"(pb));
  cf r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(pr));
  return r;
#else
  return mk(a.x + b.x, a.y + b.y);
#endif
}
__device__ __forceinline__ cf operator-(cf a, cf b) {
#if CSSM_F32X2
  unsigned long long pa, pb, pr;
  asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(pb) : "f"(b.x), "f"(b.y));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(pr) : "l"(pa), "l"(pb));
  cf r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(pr));
  return r;
#else
  return mk(a.x - b.x, a.y - b.y);
#endif
}
__device__ __forceinline__ cf cmul(cf a, cf b) {
  return mk(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
// a * conj(b)
__device__ __forceinline__ cf cmulc(cf a, cf b) {
  return mk(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
// SiLU / sigmoid through a reciprocal instead of an IEEE division: the division's slow path
// (taken for zero or denormal numerators, which real activations are full of) costs several
// times the fast path.  rcp.approx is within 1 ulp; far inside the block's 1e-4 tolerance.
__device__ __forceinline__ float rcp_fast(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}
__device__ __forceinline__ float silu_f(float v) { return v * rcp_fast(1.0f + __expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return rcp_fast(1.0f + __expf(-v)); }

// Host-side record of the last CUDA error seen on this thread.
void set_cuda_error(cudaError_t e);
int check_launch();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- plan layouts (device memory prepared by *_plan_init) ----
struct GatedPlan {
  size_t khat;     // cf [C][H*Wf] in the bin order of the spectral kernel in use
  size_t rope_t;   // float2 [T][C/2]  (cos, sin)
  size_t rope_h;   // float2 [H][C/2]
  size_t rope_w;   // float2 [W][C/2]
  size_t rope_nz;  // float  [C/2]  1 = pair rotated on some axis, 0 = angle identically zero
  size_t total;
};
GatedPlan gated_plan_layout(const cssm_gated_desc& d);

// Which spectral kernel handles an (H, W) plane.
enum SpectralPath { PATH_GENERIC = 0, PATH_R64 = 1, PATH_R32 = 2 };
SpectralPath spectral_path(int H, int W);

// Position of frequency bin (kh, kw) inside a per-(b,t) gate map / per-channel K_hat.
__host__ __device__ inline int bin_index(int path, int kh, int kw, int H, int Wf) {
  if (path == PATH_R64) return (((kh >> 3) * 33 + kw) << 3) + (kh & 7);
  if (path == PATH_R32) return ((((((kh >> 2) & 1) << 2) | (kh >> 3)) * 17 + kw) << 2) + (kh & 3);
  return kh * Wf + kw;
}

}  // namespace cssm
