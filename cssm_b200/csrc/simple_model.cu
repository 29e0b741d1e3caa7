// SimpleCSSM model around one block: stem kernels, readout kernels and the extern "C" drivers.
//   stem   : per layer conv (3x3 'SAME' or 1x1) + bias -> softplus -> LayerNorm over channels
//            -> 2x2 max-pool (default stem only), one fused kernel per layer
//   readout: (block output's last frame + residual frame) -> LayerNorm/softplus -> spatial pool
//            -> LayerNorm -> Dense head
// Reference: src/models/simple_cssm.py:244-281 (stem), 482 (residual), 523-556 (readout).
#include <string.h>
#include "kernels.cuh"

namespace cssm {

constexpr int SM_MAXC = 64;          // embed_dim limit (channel vectors live in registers)
constexpr int STEM_THREADS = 256;

__device__ __forceinline__ float softplus_f(float a) {
  return fmaxf(a, 0.f) + __logf(1.0f + __expf(-fabsf(a)));
}

// LayerNorm over the C values of v (eps 1e-6, variance as E[d^2] - E[d]^2 of d = v - v[0]), in place.
__device__ __forceinline__ void layer_norm_regs(float (&v)[SM_MAXC], int C, const float* __restrict__ scale,
                                                const float* __restrict__ bias) {
  // moments of v - v[0] (same mean-centred values and variance): a pixel whose channels are all
  // equal then normalises to exactly zero, where a plain fp32 sum leaves a 1-ulp residue that the
  // 1e-6 epsilon magnifies a thousandfold
  const float vref = v[0];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int c = 0; c < SM_MAXC; ++c)
    if (c < C) { v[c] -= vref; s += v[c]; ss = fmaf(v[c], v[c], ss); }
  const float mean = s / (float)C;
  const float var = fmaxf(ss / (float)C - mean * mean, 0.f);
  const float rinv = rsqrtf(var + 1e-6f);
#pragma unroll
  for (int c = 0; c < SM_MAXC; ++c)
    if (c < C) v[c] = (v[c] - mean) * rinv * scale[c] + bias[c];
}

struct StemArgs {
  const float* x; float* out;           // (N,Hin,Win,Cin) -> (N,Ho,Wo,C), channels-last
  const float* wk; const float* bk;     // (KS,KS,Cin,C), (C)
  const float* scale; const float* bias;
  int N, Hin, Win, Cin, C, Ho, Wo;
  int w_in_smem;                        // conv kernel staged in shared memory
};

// Four lanes share one pre-pool pixel: lane g of the quad owns the float4 channel groups
// j = g + 4k (k = 0..3, j < C/4), i.e. channels 4j..4j+3.  LayerNorm sums cross the quad by two
// shuffles.  With pooling the four pixels of a 2x2 window sit in the same warp (lane bits 2-3),
// the maximum crosses them by two more shuffles per value, and window pixel k stores group
// g + 4k, so every lane issues one 16-byte store and a quad writes 64 contiguous bytes.
//   POOL = 2: lane = g | dq << 2 | window << 4   (2 windows per warp, 16 per CTA)
//   POOL = 1: lane = g | pixel << 2              (8 pixels per warp, 64 per CTA)
// CIN > 0: compile-time input channel count (the tap loops unroll fully, so all input loads of
// a pixel are in flight together); CIN = 0: run-time a.Cin.
// FULLC: C == 64, every lane's four channel groups are live (no run-time group checks).
// NT: threads per CTA.  256 by default; 1024 when the conv weights fill most of the shared memory
// (a 64 -> 64 channel 3x3 layer: 147 KB), so that the one resident CTA still has 32 warps.
template <int KS, int POOL, int CIN, bool FULLC, int NT>
__global__ void __launch_bounds__(NT) stem_layer_kernel(const StemArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int C = FULLC ? SM_MAXC : a.C, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Cin = CIN > 0 ? CIN : a.Cin;
  const int nw = KS * KS * Cin * C;
  float* wsm = sm;                                   // [tap][ci][C] when w_in_smem
  float* vec = sm + (a.w_in_smem ? nw : 0);          // bias, scale, lnbias
  if (a.w_in_smem)
    for (int i = tid; i < nw; i += NT) wsm[i] = a.wk[i];
  for (int i = tid; i < C; i += NT) {
    vec[i] = a.bk[i]; vec[C + i] = a.scale[i]; vec[2 * C + i] = a.bias[i];
  }
  __syncthreads();
  const float* wsrc = a.w_in_smem ? wsm : a.wk;
  const int g = lane & 3, ngrp = FULLC ? SM_MAXC / 4 : C >> 2;
  const long long total = (long long)a.N * a.Ho * a.Wo;
  constexpr int WARPS = NT / 32;
  const int dq = POOL == 2 ? (lane >> 2) & 3 : 0;
  constexpr int PER_WARP = POOL == 2 ? 2 : 8;        // output pixels per warp and iteration
  // grid-stride over groups of PER_WARP output pixels; the trip count is the same for all lanes
  for (long long grp = (long long)blockIdx.x * WARPS + warp; grp * PER_WARP < total;
       grp += (long long)gridDim.x * WARPS) {
  const long long o = grp * PER_WARP + (POOL == 2 ? (lane >> 4) : (lane >> 2));
  const bool valid = o < total;
  const long long oc = valid ? o : 0;
  const int wo = (int)(oc % a.Wo), ho = (int)((oc / a.Wo) % a.Ho), n = (int)(oc / ((long long)a.Wo * a.Ho));
  const int h = ho * POOL + (dq >> 1), w = wo * POOL + (dq & 1);
  const bool inb = valid && h < a.Hin && w < a.Win;   // false: 'SAME' pool padding on odd sizes
  constexpr int LO = (KS - 1) / 2;
  float acc[4][4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int j = g + 4 * k;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[k][e] = j < ngrp ? vec[4 * j + e] : 0.f;
  }
  auto tap_ci = [&](const float4* w4, int ci, float xv) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = g + 4 * k;
      if (j < ngrp) {
        const float4 wv = w4[ci * ngrp + j];
        acc[k][0] = fmaf(xv, wv.x, acc[k][0]);
        acc[k][1] = fmaf(xv, wv.y, acc[k][1]);
        acc[k][2] = fmaf(xv, wv.z, acc[k][2]);
        acc[k][3] = fmaf(xv, wv.w, acc[k][3]);
      }
    }
  };
  if (CIN > 0) {
    // all taps' inputs first (zero outside the frame: a zero input adds nothing), then the FMAs
    float xin[KS * KS * (CIN > 0 ? CIN : 1)];
#pragma unroll
    for (int tap = 0; tap < KS * KS; ++tap) {
      const int hh = h + tap / KS - LO, ww = w + tap % KS - LO;
      const bool ok = inb && hh >= 0 && hh < a.Hin && ww >= 0 && ww < a.Win;
      const float* xp = a.x + (((size_t)n * a.Hin + (ok ? hh : 0)) * a.Win + (ok ? ww : 0)) * Cin;
#pragma unroll
      for (int ci = 0; ci < (CIN > 0 ? CIN : 1); ++ci) xin[tap * (CIN > 0 ? CIN : 1) + ci] = ok ? __ldg(xp + ci) : 0.f;
    }
#pragma unroll
    for (int tap = 0; tap < KS * KS; ++tap) {
      const float4* w4 = reinterpret_cast<const float4*>(wsrc + (size_t)tap * Cin * C);
#pragma unroll
      for (int ci = 0; ci < (CIN > 0 ? CIN : 1); ++ci) tap_ci(w4, ci, xin[tap * (CIN > 0 ? CIN : 1) + ci]);
    }
  } else if (inb) {
#pragma unroll 1
    for (int tap = 0; tap < KS * KS; ++tap) {
      const int hh = h + tap / KS - LO, ww = w + tap % KS - LO;
      if (hh < 0 || hh >= a.Hin || ww < 0 || ww >= a.Win) continue;
      const float* xp = a.x + (((size_t)n * a.Hin + hh) * a.Win + ww) * Cin;
      const float4* w4 = reinterpret_cast<const float4*>(wsrc + (size_t)tap * Cin * C);
      // float4 input reads when the channel count allows (it does for embed_dim inputs)
      if ((Cin & 3) == 0) {
#pragma unroll 2
        for (int c4 = 0; c4 < Cin; c4 += 4) {
          const float4 xv = __ldg(reinterpret_cast<const float4*>(xp + c4));
          tap_ci(w4, c4, xv.x); tap_ci(w4, c4 + 1, xv.y); tap_ci(w4, c4 + 2, xv.z); tap_ci(w4, c4 + 3, xv.w);
        }
      } else {
        for (int ci = 0; ci < Cin; ++ci) tap_ci(w4, ci, __ldg(xp + ci));
      }
    }
  }
  // softplus, then LayerNorm over the C channels of the pixel (the quad's 4 x 16 values)
  // (moments of the values minus the pixel's first channel: see layer_norm_regs)
  float s = 0.f, ss = 0.f;
  const float vref = __shfl_sync(0xffffffffu, softplus_f(acc[0][0]), lane & ~3);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (g + 4 * k < ngrp) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = softplus_f(acc[k][e]) - vref;
        acc[k][e] = v; s += v; ss = fmaf(v, v, ss);
      }
    }
  s += __shfl_xor_sync(0xffffffffu, s, 1);  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  const float mean = s / (float)C;
  const float rinv = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + 1e-6f);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int j = g + 4 * k;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v = -INFINITY;
      if (inb && j < ngrp) v = (acc[k][e] - mean) * rinv * vec[C + 4 * j + e] + vec[2 * C + 4 * j + e];
      if (POOL == 2) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      }
      acc[k][e] = v;
    }
  }
  float4* op = reinterpret_cast<float4*>(a.out + (size_t)oc * C);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int j = g + 4 * k;
    if (valid && j < ngrp && (POOL == 1 || k == dq))
      op[j] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
  }
  }
}

// Stem layer with many input channels (the second and later layers: Cin = embed_dim).  The conv
// weights (K*K*Cin*C floats, 147 KB at 3x3x64x64) fill most of the shared memory and every FMA
// needs one of them, so the kernel is bound by shared-memory reads unless a weight is reused: here
// a lane owns ALL FOUR pixels of a 2x2 pool window (for its float4 channel groups g + 4k), loads a
// weight float4 once and uses it for the four pixels; the max-pool then needs no shuffles.
// lane = g | window << 2 (8 windows per warp).  One CTA of 512 threads per SM loops over windows.
constexpr int STEMW_THREADS = 512;
template <int KS>
__global__ void __launch_bounds__(STEMW_THREADS) stem_layer_wide_kernel(const StemArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int C = a.C, Cin = a.Cin, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nw = KS * KS * Cin * C;
  float* wsm = sm;
  float* vec = sm + nw;
  for (int i = tid; i < nw; i += STEMW_THREADS) wsm[i] = a.wk[i];
  for (int i = tid; i < C; i += STEMW_THREADS) {
    vec[i] = a.bk[i]; vec[C + i] = a.scale[i]; vec[2 * C + i] = a.bias[i];
  }
  __syncthreads();
  const int g = lane & 3, ngrp = C >> 2;
  constexpr int LO = (KS - 1) / 2, WARPS = STEMW_THREADS / 32;
  const long long total = (long long)a.N * a.Ho * a.Wo;
  for (long long grp = (long long)blockIdx.x * WARPS + warp; grp * 8 < total;
       grp += (long long)gridDim.x * WARPS) {
    const long long o = grp * 8 + (lane >> 2);
    const bool valid = o < total;
    const long long oc = valid ? o : 0;
    const int wo = (int)(oc % a.Wo), ho = (int)((oc / a.Wo) % a.Ho), n = (int)(oc / ((long long)a.Wo * a.Ho));
    float acc[4][4][4];                               // [window pixel][group k][element]
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int j = g + 4 * k;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[p][k][e] = j < ngrp ? vec[4 * j + e] : 0.f;
      }
    if (valid) {
#pragma unroll 1
      for (int tap = 0; tap < KS * KS; ++tap) {
        const float* xp[4];
        bool ok[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const int hh = 2 * ho + (p >> 1) + tap / KS - LO, ww = 2 * wo + (p & 1) + tap % KS - LO;
          ok[p] = hh >= 0 && hh < a.Hin && ww >= 0 && ww < a.Win;
          xp[p] = a.x + (((size_t)n * a.Hin + (ok[p] ? hh : 0)) * a.Win + (ok[p] ? ww : 0)) * Cin;
        }
        const float4* w4 = reinterpret_cast<const float4*>(wsm + (size_t)tap * Cin * C);
#pragma unroll 1
        for (int c4 = 0; c4 < Cin; c4 += 4) {
          float xv[4][4];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const float4 t = ok[p] ? __ldg(reinterpret_cast<const float4*>(xp[p] + c4))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            xv[p][0] = t.x; xv[p][1] = t.y; xv[p][2] = t.z; xv[p][3] = t.w;
          }
#pragma unroll
          for (int ci = 0; ci < 4; ++ci)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int j = g + 4 * k;
              if (j < ngrp) {
                const float4 wv = w4[(c4 + ci) * ngrp + j];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                  acc[p][k][0] = fmaf(xv[p][ci], wv.x, acc[p][k][0]);
                  acc[p][k][1] = fmaf(xv[p][ci], wv.y, acc[p][k][1]);
                  acc[p][k][2] = fmaf(xv[p][ci], wv.z, acc[p][k][2]);
                  acc[p][k][3] = fmaf(xv[p][ci], wv.w, acc[p][k][3]);
                }
              }
            }
        }
      }
    }
    // per window pixel: softplus, LayerNorm over the quad's channels; running max over the pixels
    float mx[4][4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[k][e] = -INFINITY;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float s = 0.f, ss = 0.f;
      const float vref = __shfl_sync(0xffffffffu, softplus_f(acc[p][0][0]), lane & ~3);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (g + 4 * k < ngrp) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = softplus_f(acc[p][k][e]) - vref;
            acc[p][k][e] = v; s += v; ss = fmaf(v, v, ss);
          }
        }
      s += __shfl_xor_sync(0xffffffffu, s, 1);  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float mean = s / (float)C;
      const float rinv = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + 1e-6f);
      const bool inb = 2 * ho + (p >> 1) < a.Hin && 2 * wo + (p & 1) < a.Win;   // else pool padding
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int j = g + 4 * k;
        if (inb && j < ngrp) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            mx[k][e] = fmaxf(mx[k][e], (acc[p][k][e] - mean) * rinv * vec[C + 4 * j + e] + vec[2 * C + 4 * j + e]);
        }
      }
    }
    float4* op = reinterpret_cast<float4*>(a.out + (size_t)oc * C);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = g + 4 * k;
      if (valid && j < ngrp) op[j] = make_float4(mx[k][0], mx[k][1], mx[k][2], mx[k][3]);
    }
  }
}

template <int KS>
static int launch_stem_layer_wide(StemArgs a, cudaStream_t st) {
  const size_t smem = ((size_t)KS * KS * a.Cin * a.C + 3 * (size_t)a.C) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(stem_layer_wide_kernel<KS>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const long long total = (long long)a.N * a.Ho * a.Wo;
  const long long per_cta = (STEMW_THREADS / 32) * 8;
  const long long need = (total + per_cta - 1) / per_cta;
  stem_layer_wide_kernel<KS><<<(unsigned)(need < 148 ? need : 148), STEMW_THREADS, smem, st>>>(a);
  return check_launch();
}

template <int KS, int POOL, int CIN, bool FULLC, int NT>
static int launch_stem_layer_v(StemArgs a, cudaStream_t st) {
  const size_t wbytes = (size_t)KS * KS * a.Cin * a.C * sizeof(float);
  a.w_in_smem = wbytes <= 160 * 1024 ? 1 : 0;
  const size_t smem = (a.w_in_smem ? wbytes : 0) + 3 * (size_t)a.C * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(stem_layer_kernel<KS, POOL, CIN, FULLC, NT>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const long long total = (long long)a.N * a.Ho * a.Wo;
  const long long per_cta = (NT / 32) * (POOL == 2 ? 2 : 8);
  const long long need = (total + per_cta - 1) / per_cta;
  // a few resident waves of CTAs that loop, so that the per-CTA weight staging is amortised
  const long long cap = NT == 1024 ? 148 : 148 * 16;
  const unsigned grid = (unsigned)(need < cap ? need : cap);
  stem_layer_kernel<KS, POOL, CIN, FULLC, NT><<<grid, NT, smem, st>>>(a);
  return check_launch();
}

template <int KS, int POOL, int CIN>
static int launch_stem_layer_cin(const StemArgs& a, cudaStream_t st) {
  // many input channels, pooled: the weight-reusing kernel (needs the weights in shared memory
  // and float4 input reads)
  const size_t wbytes = (size_t)KS * KS * a.Cin * a.C * sizeof(float);
  // it needs one full wave of windows to pay (measured at 64 -> 64 channels on 128x128 images:
  // batch 8: 0.20 ms narrow vs 0.24 ms wide; batch 128: 2.67 vs 1.71 ms, both layers)
  const long long windows = (long long)a.N * a.Ho * a.Wo;
  if (CIN == 0 && POOL == 2 && a.Cin % 4 == 0 && a.Cin >= 16 && wbytes <= 200 * 1024 &&
      windows >= 148LL * (STEMW_THREADS / 32) * 8)
    return launch_stem_layer_wide<KS>(a, st);
  // otherwise: weights beyond 64 KB leave room for one CTA per SM only, give that CTA 32 warps
  if (CIN == 0 && wbytes > 64 * 1024)
    return a.C == SM_MAXC ? launch_stem_layer_v<KS, POOL, 0, true, 1024>(a, st)
                          : launch_stem_layer_v<KS, POOL, 0, false, 1024>(a, st);
  return a.C == SM_MAXC ? launch_stem_layer_v<KS, POOL, CIN, true, STEM_THREADS>(a, st)
                        : launch_stem_layer_v<KS, POOL, CIN, false, STEM_THREADS>(a, st);
}

template <int KS, int POOL>
static int launch_stem_layer(const StemArgs& a, cudaStream_t st) {
  if (a.Cin == 1) return launch_stem_layer_cin<KS, POOL, 1>(a, st);
  if (a.Cin == 3) return launch_stem_layer_cin<KS, POOL, 3>(a, st);
  return launch_stem_layer_cin<KS, POOL, 0>(a, st);
}

// ------------------------------------------------------------------------- readout ----
constexpr int RO_THREADS = 256, RO_ROWS = 8;

struct ReadoutArgs {
  const float* y; size_t y_stride;      // block output's last frame, per batch element
  const float* res; size_t res_stride;  // residual frame
  const float* pre_scale; const float* pre_bias;
  const float* post_scale; const float* post_bias;
  const float* head_k; const float* head_b;
  float* partial; float* logits;
  int B, H, W, C, pool_max, norm_post_order, ncls, bands;
};

// grid (bands, B): LayerNorm/softplus of (y + res) per pixel, pooled over the band's pixels.
// Four lanes per pixel as in the stem (lane g owns float4 groups g + 4k); 8 pixels per warp.
__global__ void __launch_bounds__(RO_THREADS) readout_pool_kernel(const ReadoutArgs a) {
  __shared__ float red[RO_THREADS / 32][SM_MAXC];
  __shared__ float vec[2 * SM_MAXC];
  const int C = a.C, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int band = blockIdx.x, b = blockIdx.y;
  for (int i = tid; i < C; i += RO_THREADS) { vec[i] = a.pre_scale[i]; vec[SM_MAXC + i] = a.pre_bias[i]; }
  __syncthreads();
  const int g = lane & 3, ps = lane >> 2, ngrp = C >> 2;
  const int h0 = band * RO_ROWS, rows = min(RO_ROWS, a.H - h0);
  const int npx = rows * a.W;
  const float init = a.pool_max ? -INFINITY : 0.f;
  float pool[4][4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int e = 0; e < 4; ++e) pool[k][e] = init;
  for (int p0 = warp * 8; p0 < npx; p0 += (RO_THREADS / 32) * 8) {      // uniform per warp
    const int p = p0 + ps;
    const bool on = p < npx;
    const size_t px = (size_t)h0 * a.W + (on ? p : 0);
    const float4* yp = reinterpret_cast<const float4*>(a.y + (size_t)b * a.y_stride + px * C);
    const float4* rp = reinterpret_cast<const float4*>(a.res + (size_t)b * a.res_stride + px * C);
    float v[4][4];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = g + 4 * k;
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < ngrp) {
        const float4 yv = __ldg(yp + j), rv = __ldg(rp + j);
        t = make_float4(yv.x + rv.x, yv.y + rv.y, yv.z + rv.z, yv.w + rv.w);
        if (a.norm_post_order) t = make_float4(softplus_f(t.x), softplus_f(t.y), softplus_f(t.z), softplus_f(t.w));
      }
      v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
    }
    // moments of the values minus the pixel's first channel (see layer_norm_regs)
    const float vref = __shfl_sync(0xffffffffu, v[0][0], lane & ~3);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (g + 4 * k < ngrp) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { v[k][e] -= vref; s += v[k][e]; ss = fmaf(v[k][e], v[k][e], ss); }
      }
    s += __shfl_xor_sync(0xffffffffu, s, 1);  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    const float mean = s / (float)C;
    const float rinv = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + 1e-6f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int j = g + 4 * k;
      if (on && j < ngrp) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = (v[k][e] - mean) * rinv * vec[4 * j + e] + vec[SM_MAXC + 4 * j + e];
          if (!a.norm_post_order) x = softplus_f(x);
          pool[k][e] = a.pool_max ? fmaxf(pool[k][e], x) : pool[k][e] + x;
        }
      }
    }
  }
  // over the warp's 8 pixel slots, then over the warps
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float r = pool[k][e];
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, r, off);
        r = a.pool_max ? fmaxf(r, o) : r + o;
      }
      const int j = g + 4 * k;
      if (ps == 0 && j < ngrp) red[warp][4 * j + e] = r;
    }
  __syncthreads();
  if (tid < C) {
    float r = red[0][tid];
    for (int w = 1; w < RO_THREADS / 32; ++w) r = a.pool_max ? fmaxf(r, red[w][tid]) : r + red[w][tid];
    a.partial[((size_t)b * a.bands + band) * C + tid] = r;
  }
}

// grid B, 64 threads: combine the band partials, LayerNorm (norm_post), Dense head
__global__ void __launch_bounds__(SM_MAXC) readout_head_kernel(const ReadoutArgs a) {
  __shared__ float v[SM_MAXC];
  __shared__ float stats[2];
  const int C = a.C, tid = threadIdx.x, b = blockIdx.x;
  float r = 0.f;
  if (tid < C) {
    r = a.partial[(size_t)b * a.bands * C + tid];
    for (int k = 1; k < a.bands; ++k) {
      const float o = a.partial[((size_t)b * a.bands + k) * C + tid];
      r = a.pool_max ? fmaxf(r, o) : r + o;
    }
    if (!a.pool_max) r /= (float)(a.H * a.W);
    v[tid] = r;
  }
  __syncthreads();
  if (tid == 0) {
    float s = 0.f, ss = 0.f;
    const float vref = v[0];
    for (int c = 0; c < C; ++c) { const float d = v[c] - vref; s += d; ss = fmaf(d, d, ss); }
    const float mean = s / (float)C;
    stats[0] = mean + vref;
    stats[1] = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + 1e-6f);
  }
  __syncthreads();
  if (tid < C) v[tid] = (v[tid] - stats[0]) * stats[1] * a.post_scale[tid] + a.post_bias[tid];
  __syncthreads();
  if (tid < a.ncls) {
    float acc = a.head_b[tid];
    for (int c = 0; c < C; ++c) acc = fmaf(v[c], a.head_k[(size_t)c * a.ncls + tid], acc);
    a.logits[(size_t)b * a.ncls + tid] = acc;
  }
}

// ------------------------------------------------------------------- host helpers ----
struct SimpleDims { int N, H, W; };   // stem output: N frames of H x W x embed_dim

static int simple_validate(const cssm_simple_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->Hin <= 0 || d->Win <= 0 || d->Cin <= 0 || d->num_classes <= 0)
    return CSSM_ERR_DIMS;
  if (d->embed_dim <= 0 || d->embed_dim % 4 != 0 || d->embed_dim > SM_MAXC) return CSSM_ERR_UNSUPPORTED;
  if (d->num_classes > SM_MAXC) return CSSM_ERR_UNSUPPORTED;
  if (d->stem_mode != 0 && d->stem_mode != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->stem_mode == 0 && (d->stem_layers < 1 || d->stem_layers > 4)) return CSSM_ERR_UNSUPPORTED;
  if (d->block < 0 || d->block > 4) return CSSM_ERR_UNSUPPORTED;
  if (d->pool_type != 0 && d->pool_type != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->readout_norm != 0 && d->readout_norm != 1) return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

static SimpleDims stem_out_dims(const cssm_simple_desc& d) {
  SimpleDims o;
  o.N = d.image_input ? d.B : d.B * d.T;
  o.H = d.Hin; o.W = d.Win;
  if (d.stem_mode == 0)
    for (int i = 0; i < d.stem_layers; ++i) { o.H = (o.H + 1) / 2; o.W = (o.W + 1) / 2; }
  return o;
}

// every block descriptor starts with int32 B, T, H, W, C
struct BlockDims { int32_t B, T, H, W, C; };
static bool block_matches(const cssm_simple_desc& d, const void* bd) {
  const SimpleDims o = stem_out_dims(d);
  const BlockDims* g = (const BlockDims*)bd;
  return g->B == d.B && g->T == d.T && g->H == o.H && g->W == o.W && g->C == d.embed_dim;
}

static size_t block_ws_bytes(int block, const void* bd) {
  switch (block) {
    case 0: return cssm_gated_workspace_bytes((const cssm_gated_desc*)bd);
    case 1: return cssm_gdn_workspace_bytes((const cssm_gdn_desc*)bd);
    case 2: return cssm_nogate_workspace_bytes((const cssm_nogate_desc*)bd);
    case 3: return cssm_additive_workspace_bytes((const cssm_additive_desc*)bd);
    default: return cssm_deltanet_workspace_bytes((const cssm_deltanet_desc*)bd);
  }
}

// one feature frame per image -> T equal frames per clip (the scalar-scan blocks read clips)
__global__ void __launch_bounds__(256) repeat_frames_kernel(const float4* __restrict__ in,
                                                            float4* __restrict__ out, size_t frame4,
                                                            int T, size_t total4) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total4) return;
  const size_t fo = i / frame4, r = i - fo * frame4;
  out[i] = __ldg(in + (fo / T) * frame4 + r);
}

struct SimpleWs { size_t feat, tmp, y, partial, rep, block, total; };
static SimpleWs simple_ws_layout(const cssm_simple_desc& d, const void* bd) {
  SimpleWs l;
  const SimpleDims o = stem_out_dims(d);
  const size_t C = d.embed_dim;
  const size_t N = o.N;
  size_t off = 0;
  l.feat = off; off += round_up(N * o.H * o.W * C * sizeof(float), 256);
  // ping-pong buffers of a multi-layer stem: the first layer's output is the largest
  size_t tmp = 0;
  if (d.stem_mode == 0 && d.stem_layers > 1)
    tmp = N * ((d.Hin + 1) / 2) * ((d.Win + 1) / 2) * C * sizeof(float);
  l.tmp = off; off += 2 * round_up(tmp, 256);
  l.y = off; off += round_up((size_t)d.B * d.T * o.H * o.W * C * sizeof(float), 256);
  l.partial = off; off += round_up((size_t)d.B * ((o.H + RO_ROWS - 1) / RO_ROWS) * C * sizeof(float), 256);
  // blocks 2..4 take clips only: an image batch's features are repeated over T for them
  l.rep = off;
  if (d.block >= 2 && d.image_input) off += round_up((size_t)d.B * d.T * o.H * o.W * C * sizeof(float), 256);
  l.block = off;
  off += block_ws_bytes(d.block, bd);
  l.total = round_up(off, 256);
  return l;
}

static int run_stem(const cssm_simple_desc* d, const cssm_simple_weights* w, const float* x,
                    float* feat, float* tmp0, float* tmp1, cudaStream_t st) {
  StemArgs a;
  memset(&a, 0, sizeof(a));
  a.N = d->image_input ? d->B : d->B * d->T;
  a.C = d->embed_dim;
  if (d->stem_mode == 1) {
    if (!w->conv_kernel[0] || !w->conv_bias[0] || !w->norm_scale[0] || !w->norm_bias[0]) return CSSM_ERR_NULL;
    a.x = x; a.out = feat; a.wk = w->conv_kernel[0]; a.bk = w->conv_bias[0];
    a.scale = w->norm_scale[0]; a.bias = w->norm_bias[0];
    a.Hin = d->Hin; a.Win = d->Win; a.Cin = d->Cin; a.Ho = d->Hin; a.Wo = d->Win;
    return launch_stem_layer<1, 1>(a, st);
  }
  const float* src = x;
  int H = d->Hin, W = d->Win, Cin = d->Cin;
  for (int i = 0; i < d->stem_layers; ++i) {
    if (!w->conv_kernel[i] || !w->conv_bias[i] || !w->norm_scale[i] || !w->norm_bias[i]) return CSSM_ERR_NULL;
    const bool last = i == d->stem_layers - 1;
    float* dst = last ? feat : ((i & 1) ? tmp1 : tmp0);
    a.x = src; a.out = dst; a.wk = w->conv_kernel[i]; a.bk = w->conv_bias[i];
    a.scale = w->norm_scale[i]; a.bias = w->norm_bias[i];
    a.Hin = H; a.Win = W; a.Cin = Cin; a.Ho = (H + 1) / 2; a.Wo = (W + 1) / 2;
    const int s = launch_stem_layer<3, 2>(a, st);
    if (s != CSSM_OK) return s;
    src = dst; H = a.Ho; W = a.Wo; Cin = d->embed_dim;
  }
  return CSSM_OK;
}

static int run_readout(const cssm_simple_desc* d, const cssm_simple_weights* w, int H, int W,
                       const float* y, size_t ys, const float* res, size_t rs, float* partial,
                       float* logits, cudaStream_t st) {
  if (!w->norm_pre_scale || !w->norm_pre_bias || !w->norm_post_scale || !w->norm_post_bias ||
      !w->head_kernel || !w->head_bias)
    return CSSM_ERR_NULL;
  ReadoutArgs a;
  memset(&a, 0, sizeof(a));
  a.y = y; a.y_stride = ys; a.res = res; a.res_stride = rs;
  a.pre_scale = w->norm_pre_scale; a.pre_bias = w->norm_pre_bias;
  a.post_scale = w->norm_post_scale; a.post_bias = w->norm_post_bias;
  a.head_k = w->head_kernel; a.head_b = w->head_bias;
  a.partial = partial; a.logits = logits;
  a.B = d->B; a.H = H; a.W = W; a.C = d->embed_dim; a.pool_max = d->pool_type;
  a.norm_post_order = d->readout_norm; a.ncls = d->num_classes;
  a.bands = (H + RO_ROWS - 1) / RO_ROWS;
  readout_pool_kernel<<<dim3(a.bands, d->B), RO_THREADS, 0, st>>>(a);
  int s = check_launch();
  if (s != CSSM_OK) return s;
  readout_head_kernel<<<d->B, SM_MAXC, 0, st>>>(a);
  return check_launch();
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_simple_workspace_bytes(const cssm_simple_desc* d, const void* block_desc) {
  if (simple_validate(d) != CSSM_OK || !block_desc || !block_matches(*d, block_desc)) return 0;
  // a block descriptor its own library entry points reject makes the model unsupported too
  const size_t bws = block_ws_bytes(d->block, block_desc);
  if (bws == 0) return 0;
  return simple_ws_layout(*d, block_desc).total;
}

int cssm_simple_stem(const cssm_simple_desc* d, const cssm_simple_weights* w, const float* x,
                     float* feat, void* workspace, size_t workspace_bytes, void* stream) {
  int s = simple_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !x || !feat) return CSSM_ERR_NULL;
  if (!aligned16(x) || !aligned16(feat)) return CSSM_ERR_ALIGN;
  float* t0 = nullptr;
  float* t1 = nullptr;
  if (d->stem_mode == 0 && d->stem_layers > 1) {
    const SimpleDims o = stem_out_dims(*d);
    const size_t tmp = round_up((size_t)o.N * ((d->Hin + 1) / 2) * ((d->Win + 1) / 2) * d->embed_dim * sizeof(float), 256);
    if (!workspace) return CSSM_ERR_NULL;
    if (!aligned16(workspace)) return CSSM_ERR_ALIGN;
    if (workspace_bytes < 2 * tmp) return CSSM_ERR_WORKSPACE;
    t0 = (float*)workspace; t1 = (float*)((char*)workspace + tmp);
  }
  return run_stem(d, w, x, feat, t0, t1, (cudaStream_t)stream);
}

int cssm_simple_readout(const cssm_simple_desc* d, const cssm_simple_weights* w, int32_t H,
                        int32_t W, const float* y_last, size_t y_stride, const float* res,
                        size_t res_stride, float* partial, float* logits, void* stream) {
  int s = simple_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !y_last || !res || !partial || !logits) return CSSM_ERR_NULL;
  if (H <= 0 || W <= 0) return CSSM_ERR_DIMS;
  if (!aligned16(y_last) || !aligned16(res) || y_stride % 4 != 0 || res_stride % 4 != 0) return CSSM_ERR_ALIGN;
  return run_readout(d, w, H, W, y_last, y_stride, res, res_stride, partial, logits, (cudaStream_t)stream);
}

int cssm_simple_forward(const cssm_simple_desc* d, const cssm_simple_weights* w,
                        const void* block_desc, const void* block_weights, const void* block_plan,
                        const float* x, float* logits, void* workspace, size_t workspace_bytes,
                        int32_t flags, void* stream) {
  int s = simple_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !block_desc || !block_weights || !block_plan || !x || !logits || !workspace) return CSSM_ERR_NULL;
  if (!block_matches(*d, block_desc)) return CSSM_ERR_DIMS;
  if (!aligned16(x) || !aligned16(workspace)) return CSSM_ERR_ALIGN;
  const SimpleWs l = simple_ws_layout(*d, block_desc);
  if (workspace_bytes < l.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  const SimpleDims o = stem_out_dims(*d);
  float* feat = (float*)(ws + l.feat);
  float* y = (float*)(ws + l.y);
  const size_t tmp_half = (l.y - l.tmp) / 2;
  s = run_stem(d, w, x, feat, (float*)(ws + l.tmp), (float*)(ws + l.tmp + tmp_half), st);
  if (s != CSSM_OK) return s;
  // the scalar-scan blocks have no last-frame-only entry point: they produce all T frames
  const int last_only = ((flags & CSSM_SIMPLE_LAST_FRAME_ONLY) && d->block < 2) ? 1 : 0;
  const size_t bws = l.total - l.block;
  if (d->block >= 2) {
    const float* clips = feat;
    if (d->image_input) {
      const size_t frame4 = (size_t)o.H * o.W * d->embed_dim / 4, total4 = frame4 * d->B * d->T;
      repeat_frames_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, st>>>(
          (const float4*)feat, (float4*)(ws + l.rep), frame4, d->T, total4);
      if ((s = check_launch()) != CSSM_OK) return s;
      clips = (const float*)(ws + l.rep);
    }
    if (d->block == 2)
      s = cssm_nogate_forward((const cssm_nogate_desc*)block_desc, (const cssm_nogate_weights*)block_weights,
                              block_plan, clips, y, ws + l.block, bws, stream);
    else if (d->block == 3)
      s = cssm_additive_forward((const cssm_additive_desc*)block_desc,
                                (const cssm_additive_weights*)block_weights, block_plan, clips, y,
                                ws + l.block, bws, stream);
    else
      s = cssm_deltanet_forward((const cssm_deltanet_desc*)block_desc,
                                (const cssm_deltanet_weights*)block_weights, block_plan, clips, y,
                                ws + l.block, bws, stream);
  } else if (d->block == 0)
    s = gated_forward_internal((const cssm_gated_desc*)block_desc, (const cssm_gated_weights*)block_weights,
                               block_plan, feat, y, ws + l.block, bws, stream, last_only, d->image_input);
  else
    s = gdn_forward_internal((const cssm_gdn_desc*)block_desc, (const cssm_gdn_weights*)block_weights,
                             block_plan, feat, y, ws + l.block, bws, stream, last_only, d->image_input);
  if (s != CSSM_OK) return s;
  const size_t frame = (size_t)o.H * o.W * d->embed_dim;
  const float* y_last = last_only ? y : y + (size_t)(d->T - 1) * frame;
  const size_t ys = last_only ? frame : (size_t)d->T * frame;
  const float* res = d->image_input ? feat : feat + (size_t)(d->T - 1) * frame;
  const size_t rs = d->image_input ? frame : (size_t)d->T * frame;
  return run_readout(d, w, o.H, o.W, y_last, ys, res, rs, (float*)(ws + l.partial), logits, st);
}

size_t cssm_simple_host_workspace_bytes(const cssm_simple_desc* d, const void* block_desc) {
  const size_t base = cssm_simple_workspace_bytes(d, block_desc);
  if (base == 0) return 0;
  const size_t nx = (size_t)(d->image_input ? d->B : d->B * d->T) * d->Hin * d->Win * d->Cin * sizeof(float);
  return base + round_up(nx, 256) + round_up((size_t)d->B * d->num_classes * sizeof(float), 256);
}

int cssm_simple_forward_host(const cssm_simple_desc* d, const cssm_simple_weights* w,
                             const void* block_desc, const void* block_weights,
                             const void* block_plan, const float* x_host, float* logits_host,
                             void* workspace, size_t workspace_bytes, int32_t flags, void* stream) {
  const size_t base = cssm_simple_workspace_bytes(d, block_desc);
  if (base == 0) return simple_validate(d) != CSSM_OK ? simple_validate(d) : CSSM_ERR_DIMS;
  if (!x_host || !logits_host || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(workspace)) return CSSM_ERR_ALIGN;
  if (workspace_bytes < cssm_simple_host_workspace_bytes(d, block_desc)) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t nx = (size_t)(d->image_input ? d->B : d->B * d->T) * d->Hin * d->Win * d->Cin * sizeof(float);
  const size_t nl = (size_t)d->B * d->num_classes * sizeof(float);
  char* ws = (char*)workspace;
  float* xd = (float*)(ws + base);
  float* ld = (float*)(ws + base + round_up(nx, 256));
  cudaError_t e = cudaMemcpyAsync(xd, x_host, nx, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const int s = cssm_simple_forward(d, w, block_desc, block_weights, block_plan, xd, ld, workspace,
                                    base, flags, stream);
  if (s != CSSM_OK) return s;
  e = cudaMemcpyAsync(logits_host, ld, nl, cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

size_t cssm_simple_host_pipe_workspace_bytes(const cssm_simple_desc* d, const void* block_desc) {
  const size_t base = cssm_simple_workspace_bytes(d, block_desc);
  if (base == 0) return 0;
  const size_t nx = (size_t)(d->image_input ? d->B : d->B * d->T) * d->Hin * d->Win * d->Cin * sizeof(float);
  return base + 2 * round_up(nx, 256) + round_up((size_t)d->B * d->num_classes * sizeof(float), 256);
}

int cssm_simple_forward_host_pipelined(const cssm_simple_desc* d, const cssm_simple_weights* w,
                                       const void* block_desc, const void* block_weights,
                                       const void* block_plan, cssm_host_pipe* pipe, const float* x_host,
                                       const float* x_next_host, float* logits_host, void* workspace,
                                       size_t workspace_bytes, int32_t flags, void* stream) {
  const size_t base = cssm_simple_workspace_bytes(d, block_desc);
  if (base == 0) return simple_validate(d) != CSSM_OK ? simple_validate(d) : CSSM_ERR_DIMS;
  if (!pipe || !x_host || !logits_host || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(workspace)) return CSSM_ERR_ALIGN;
  if (workspace_bytes < cssm_simple_host_pipe_workspace_bytes(d, block_desc)) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t nx = (size_t)(d->image_input ? d->B : d->B * d->T) * d->Hin * d->Win * d->Cin * sizeof(float);
  const size_t nl = (size_t)d->B * d->num_classes * sizeof(float);
  char* ws = (char*)workspace;
  char* xb0 = ws + base;
  char* xb1 = xb0 + round_up(nx, 256);
  float* ld = (float*)(xb1 + round_up(nx, 256));
  int j = 0;
  int rc = host_pipe_stage(pipe, workspace, xb0, xb1, nx, x_host, x_next_host, st, &j);
  if (rc == CSSM_OK)
    rc = cssm_simple_forward(d, w, block_desc, block_weights, block_plan, (const float*)(j ? xb1 : xb0), ld,
                             workspace, base, flags, stream);
  if (rc == CSSM_OK) {
    const cudaError_t e = cudaMemcpyAsync(logits_host, ld, nl, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) { set_cuda_error(e); rc = CSSM_ERR_CUDA; }
  }
  const cudaError_t e1 = cudaStreamSynchronize(st);
  if (rc == CSSM_OK && e1 != cudaSuccess) { set_cuda_error(e1); rc = CSSM_ERR_CUDA; }
  if (rc != CSSM_OK) host_pipe_abort(pipe);
  return rc;
}

}  // extern "C"
