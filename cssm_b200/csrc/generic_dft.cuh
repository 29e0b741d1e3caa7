// Direct-DFT plane transforms for one CTA of GG_THREADS threads (any H, W): O(N) work per output,
// used by the kernels that cover plane sizes without a radix kernel.
#pragma once
#include "common.cuh"

namespace cssm {

constexpr int GG_THREADS = 256;

// rfft2 of one real (H, W) plane in global memory -> out[H*Wf] (shared memory).  xs: H*W floats,
// Rb: H*Wf scratch; twW[i] = e^{-2 pi i i/W}, twH[i] = e^{-2 pi i i/H}.
__device__ inline void gen_fwd_plane(const float* __restrict__ plane, float* xs, cf* Rb, cf* out,
                                     const cf* twW, const cf* twH, int H, int W) {
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf, tid = threadIdx.x;
  __syncthreads();
  for (int i = tid; i < HW; i += GG_THREADS) xs[i] = plane[i];
  __syncthreads();
  for (int o = tid; o < NB; o += GG_THREADS) {
    const int h = o / Wf, kw = o % Wf;
    float ax = 0.f, ay = 0.f;
    int idx = 0;
    for (int w = 0; w < W; ++w) {
      const cf e = twW[idx];
      const float xv = xs[h * W + w];
      ax += xv * e.x; ay += xv * e.y;
      idx += kw; if (idx >= W) idx -= W;
    }
    Rb[o] = mk(ax, ay);
  }
  __syncthreads();
  for (int o = tid; o < NB; o += GG_THREADS) {
    const int kh = o / Wf, kw = o % Wf;
    float ax = 0.f, ay = 0.f;
    int idx = 0;
    for (int h = 0; h < H; ++h) {
      const cf e = twH[idx];
      const cf r = Rb[h * Wf + kw];
      ax += r.x * e.x - r.y * e.y; ay += r.x * e.y + r.y * e.x;
      idx += kh; if (idx >= H) idx -= H;
    }
    out[o] = mk(ax, ay);
  }
}

// Unnormalised irfft2 of Fb[H*Wf] (shared memory; the caller folds in 1/(H*W)) -> real (H, W)
// plane in global memory.  The imaginary parts of the DC and Nyquist columns are ignored, as in
// a C2R transform.  Rb: H*Wf scratch.  Begins with a barrier (Fb may just have been written).
__device__ inline void gen_inv_plane(const cf* Fb, cf* Rb, float* __restrict__ plane,
                                     const cf* twW, const cf* twH, int H, int W) {
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf, tid = threadIdx.x;
  __syncthreads();
  for (int o = tid; o < NB; o += GG_THREADS) {
    const int h = o / Wf, kw = o % Wf;
    float ax = 0.f, ay = 0.f;
    int idx = 0;
    for (int kh = 0; kh < H; ++kh) {
      const cf e = twH[idx];
      const cf f = Fb[kh * Wf + kw];
      ax += f.x * e.x + f.y * e.y; ay += f.y * e.x - f.x * e.y;
      idx += h; if (idx >= H) idx -= H;
    }
    Rb[o] = mk(ax, ay);
  }
  __syncthreads();
  const int kmax = (W - 1) / 2;
  for (int o = tid; o < HW; o += GG_THREADS) {
    const int h = o / W, w = o % W;
    const cf* r = Rb + h * Wf;
    float acc = r[0].x;
    if ((W & 1) == 0) acc += (w & 1) ? -r[W / 2].x : r[W / 2].x;
    int idx = 0;
    float s2 = 0.f;
    for (int k = 1; k <= kmax; ++k) {
      idx += w; if (idx >= W) idx -= W;
      const cf e = twW[idx];
      s2 += r[k].x * e.x + r[k].y * e.y;
    }
    plane[o] = acc + 2.f * s2;
  }
}

// Sum of v over the CTA, returned to every thread.  red: one float per warp (shared memory).
__device__ inline float block_sum(float v, float* red) {
  const int tid = threadIdx.x;
  for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  return tot;
}

}  // namespace cssm
