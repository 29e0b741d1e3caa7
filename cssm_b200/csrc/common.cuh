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

// Caller-owned state of the streaming host entry points (cssm_host_pipe_create / _destroy; the type
// is opaque in the public header): one copy stream, its events, and which host buffer was prefetched
// into which of the two input buffers of which workspace.
struct cssm_host_pipe {
  cudaStream_t copy;
  cudaEvent_t copied[2];       // the copy into input buffer j has finished
  cudaEvent_t computed;        // orders a cold copy behind the work already queued on the caller's stream
  const void* src;             // host address whose batch sits (or is arriving) in buffer `buf`
  const void* ws;              // ... of this workspace
  int buf;
};

namespace cssm {
// First half of a streaming host call: makes `stream` wait for the batch x_host in input buffer
// *j of the workspace (already prefetched by the previous call on this pipe, or copied now), and
// starts the copy of x_next_host (may be null) into the other buffer on the pipe's stream.
inline int host_pipe_stage(cssm_host_pipe* p, void* workspace, char* xbuf0, char* xbuf1, size_t xbytes,
                           const void* x_host, const void* x_next_host, cudaStream_t st, int* j_out) {
  cudaError_t e = cudaSuccess;
  char* xb[2] = {xbuf0, xbuf1};
  int j;
  if (p->src == x_host && p->ws == workspace) {
    j = p->buf;                                        // prefetched by the previous call
  } else {
    j = 0;
    // after whatever the caller queued on its stream, and after any copy still running on the pipe
    e = cudaEventRecord(p->computed, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(p->copy, p->computed, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(xb[0], x_host, xbytes, cudaMemcpyHostToDevice, p->copy);
    if (e == cudaSuccess) e = cudaEventRecord(p->copied[0], p->copy);
  }
  p->src = nullptr;
  if (x_next_host != nullptr && e == cudaSuccess) {
    // buffer 1 - j was last read by the previous call's forward, which that call waited for
    e = cudaMemcpyAsync(xb[1 - j], x_next_host, xbytes, cudaMemcpyHostToDevice, p->copy);
    if (e == cudaSuccess) e = cudaEventRecord(p->copied[1 - j], p->copy);
    if (e == cudaSuccess) { p->src = x_next_host; p->ws = workspace; p->buf = 1 - j; }
  }
  if (e == cudaSuccess) e = cudaStreamWaitEvent(st, p->copied[j], 0);
  *j_out = j;
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}
// Error path of a streaming host call: leave no copy running into a workspace the caller may free.
inline void host_pipe_abort(cssm_host_pipe* p) {
  cudaStreamSynchronize(p->copy);
  p->src = nullptr;
}
}  // namespace cssm
