// Weight-only precompute (kernel spectrum, RoPE tables), the per-plane short-conv stencil
// with its plane sums, and the gate-map kernels.
#include "kernels.cuh"

namespace cssm {

// ------------------------------------------------------------ kernel spectrum ----
// K[c][kh][kw] = rfft2(centre-padded k[c]) squashed to |K| < rho, floored at 1e-7.
// One thread per bin; double precision (runs once per weight set).
__global__ void khat_kernel(const float* __restrict__ k, cf* __restrict__ out, int nch, int ks,
                            int H, int W, float rho, int squash, int floor_eps, int path) {
  const int Wf = W / 2 + 1, NB = H * Wf;
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= nch * NB) return;
  const int c = o / NB, bin = o % NB, kh = bin / Wf, kw = bin % Wf;
  // crop (ks > H or W) or centre-pad, exactly as the reference slices / pads
  int i0 = 0, i1 = ks, j0 = 0, j1 = ks, offh, offw;
  if (ks > H || ks > W) {
    const int sh = (ks - H) / 2, sw = (ks - W) / 2;
    i0 = sh; i1 = sh + H; j0 = sw; j1 = sw + W; offh = -sh; offw = -sw;
    if (i0 < 0) { i0 = 0; }
    if (j0 < 0) { j0 = 0; }
    if (i1 > ks) i1 = ks;
    if (j1 > ks) j1 = ks;
  } else {
    offh = (H - ks) / 2; offw = (W - ks) / 2;
  }
  double re = 0.0, im = 0.0;
  for (int i = i0; i < i1; ++i) {
    const int ph = i + offh;
    if (ph < 0 || ph >= H) continue;
    for (int j = j0; j < j1; ++j) {
      const int pw = j + offw;
      if (pw < 0 || pw >= W) continue;
      const double ang = -2.0 * ((double)((kh * ph) % H) / H + (double)((kw * pw) % W) / W);
      double s, co;
      sincospi(ang, &s, &co);
      const double v = k[((size_t)c * ks + i) * ks + j];
      re += v * co; im += v * s;
    }
  }
  if (squash) {
    const double mag = sqrt(re * re + im * im);
    const double sc = (double)rho / (1.0 + mag);
    re *= sc; im *= sc;
  }
  if (floor_eps && sqrt(re * re + im * im) < 1e-7) { re = 1e-7; im = 0.0; }
  out[(size_t)c * NB + bin_index(path, kh, kw, H, Wf)] = mk((float)re, (float)im);
}

int launch_khat(const float* k, cf* out, int nch, int ks, int H, int W, float rho, int squash,
                int floor_eps, int path, cudaStream_t st) {
  const int n = nch * H * (W / 2 + 1);
  khat_kernel<<<(n + 127) / 128, 128, 0, st>>>(k, out, nch, ks, H, W, rho, squash, floor_eps, path);
  return check_launch();
}

// ---------------------------------------------------------------- RoPE tables ----
// (cos, sin)(pos * f_axis[i]) for the three axes; f_axis comes from the mode exactly as
// apply_rope slices and right-pads inv_freq (cssm.py:125-244).
__device__ double rope_freq(int axis, int i, int n, int mode, double base, int C) {
  auto inv = [&](int q) { return 1.0 / pow(base, (double)(2 * q) / (double)C); };
  if (mode == CSSM_ROPE_TEMPORAL) return axis == 0 ? inv(i) : 0.0;
  if (mode == CSSM_ROPE_SPATIAL_ONLY) {
    if (axis == 1) { const int q = 2 * i; return q < n ? inv(q) : 0.0; }
    if (axis == 2) { const int q = 2 * i + 1; return q < n ? inv(q) : 0.0; }
    return 0.0;
  }
  if (mode == CSSM_ROPE_SPATIOTEMPORAL) {
    const int nt = n / 3;
    if (axis == 0) return i < nt ? inv(i) : 0.0;
    if (axis == 1) { const int q = nt + 2 * i; return q < n ? inv(q) : 0.0; }
    const int q = nt + 1 + 2 * i; return q < n ? inv(q) : 0.0;
  }
  if (mode == CSSM_ROPE_MROPE) {
    const int nt = n / 3;
    if (i < 3 * nt) {
      const int r = i % 3, q = i / 3;
      if (r != axis) return 0.0;
      return inv(axis * nt + q);
    }
    // left-over width frequencies
    return axis == 2 ? inv(2 * nt + nt + (i - 3 * nt)) : 0.0;
  }
  return 0.0;
}

__global__ void rope_table_kernel(float2* tt, float2* th, float2* tw, float* nz, int T, int H,
                                  int W, int C, int mode, float base) {
  const int n = C / 2;
  const int total = (T + H + W) * n;
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o < n) {
    // 1 where the pair is rotated on some axis, 0 where its angle is identically zero
    const bool any = rope_freq(0, o, n, mode, (double)base, C) != 0.0 ||
                     rope_freq(1, o, n, mode, (double)base, C) != 0.0 ||
                     rope_freq(2, o, n, mode, (double)base, C) != 0.0;
    nz[o] = any ? 1.f : 0.f;
  }
  if (o >= total) return;
  int pos = o / n, i = o % n, axis = 0;
  float2* dst = tt;
  if (pos >= T + H) { axis = 2; pos -= T + H; dst = tw; }
  else if (pos >= T) { axis = 1; pos -= T; dst = th; }
  const double ang = (double)pos * rope_freq(axis, i, n, mode, (double)base, C);
  dst[pos * n + i] = make_float2((float)cos(ang), (float)sin(ang));
}

int launch_rope_tables(float2* tt, float2* th, float2* tw, float* nz, int T, int H, int W, int C,
                       int mode, float base, cudaStream_t st) {
  const int total = (T + H + W) * (C / 2);
  rope_table_kernel<<<(total + 127) / 128, 128, 0, st>>>(tt, th, tw, nz, T, H, W, C, mode, base);
  return check_launch();
}

// interleaved (sin, cos) temporal code added to the GDN gate context (cssm.py:353-383)
__global__ void tcode_kernel(float* out, int T, int C, float base) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= T * C) return;
  const int t = o / C, ch = o % C, i = ch >> 1;
  const double f = 1.0 / pow((double)base, (double)(2 * i) / (double)C);
  const double ang = (double)t * f;
  out[o] = (float)((ch & 1) ? cos(ang) : sin(ang));
}

int launch_tcode(float* out, int T, int C, float base, cudaStream_t st) {
  tcode_kernel<<<(T * C + 127) / 128, 128, 0, st>>>(out, T, C, base);
  return check_launch();
}

// ------------------------------------------------------------- plane stencil ----
// One CTA per (b, channel) walks t = 0..T-1 over planes of a planar tensor, in place:
//   s_t  = dwconv_kxk(raw_t) + b_sp                (if ksp > 0, zero 'SAME' padding)
//   o_t  = b_t + sum_j w_t[j] * s_{t-(kt-1)+j}     (if kt > 0; frames before 0 are zero)
//   o_t  = silu(o_t) (if act); o_t *= post[b,t,pixel] (if post)
// and writes sum over the plane of o_t to sums[(b*T+t)*C + c] (if sums).
constexpr int ST_THREADS = 256;


// KSP / KT >= 0 fix the tap counts at compile time (taps stay in registers); -1 = run time.
template <int KSP, int KT>
__global__ void __launch_bounds__(ST_THREADS) plane_stencil_kernel(const StencilArgs s) {
  extern __shared__ __align__(16) float sm[];
  const int HW = s.H * s.W;
  float* raw = sm;                       // [HW]
  float* hist = sm + HW;                 // [(kt-1)][HW] ring of earlier s planes
  __shared__ float red[ST_THREADS / 32];
  const int tid = threadIdx.x;
  const int b = blockIdx.x / s.C, c = blockIdx.x % s.C;
  const int ksp = KSP >= 0 ? KSP : s.ksp;
  const int kt = KT >= 0 ? KT : s.kt;
  const int nh = kt > 0 ? kt - 1 : 0;

  float wsp[KSP >= 0 ? (KSP * KSP > 0 ? KSP * KSP : 1) : 49];
  if (ksp > 0) {
#pragma unroll
    for (int i = 0; i < ksp * ksp; ++i) wsp[i] = s.wsp[(size_t)i * s.C + c];
  }
  const float bsp = ksp > 0 ? s.bsp[c] : 0.f;
  float wt[KT >= 0 ? (KT > 0 ? KT : 1) : 8];
  if (kt > 0) {
#pragma unroll
    for (int j = 0; j < kt; ++j) wt[j] = s.wt[(size_t)j * s.C + c];
  }
  const float btv = kt > 0 ? s.bt[c] : 0.f;
  const int lo = (ksp - 1) / 2;

  for (int t = 0; t < s.T; ++t) {
    const size_t frame = (size_t)(b * s.T + t);
    float* p = s.buf + (frame * s.planes_per_frame + s.plane0 + c) * HW;
    __syncthreads();
    for (int i = tid; i < HW; i += ST_THREADS) raw[i] = p[i];
    __syncthreads();
    float lsum = 0.f;
    for (int i = tid; i < HW; i += ST_THREADS) {
      float v;
      if (ksp > 0) {
        const int h = i / s.W, w = i % s.W;
        v = bsp;
#pragma unroll
        for (int di = 0; di < ksp; ++di) {
          const int hh = h + di - lo;
          if (hh < 0 || hh >= s.H) continue;
#pragma unroll
          for (int dj = 0; dj < ksp; ++dj) {
            const int ww = w + dj - lo;
            if (ww < 0 || ww >= s.W) continue;
            v = fmaf(wsp[di * ksp + dj], raw[hh * s.W + ww], v);
          }
        }
      } else {
        v = raw[i];
      }
      float o = v;
      if (kt > 0) {
        o = btv + wt[kt - 1] * v;
        // tap j reads s_{t-(kt-1)+j}; ring slot of frame f is f % nh
#pragma unroll
        for (int j = 0; j < kt - 1; ++j) {
          const int f = t - (kt - 1) + j;
          if (f >= 0) o = fmaf(wt[j], hist[(f % (nh > 0 ? nh : 1)) * HW + i], o);
        }
      }
      // each thread owns pixel i in every pass, so the ring can be updated in place:
      // slot t % nh holds s_{t-nh}, which tap 0 has just consumed
      if (nh > 0) hist[(t % (nh > 0 ? nh : 1)) * HW + i] = v;
      if (s.act) o = silu_f(o);
      if (s.post) o *= s.post[(frame * HW + i) * s.post_stride + s.post_off];
      p[i] = o;
      lsum += o;
    }
    if (s.sums) {
      for (int off = 16; off > 0; off >>= 1) lsum += __shfl_down_sync(0xffffffffu, lsum, off);
      if ((tid & 31) == 0) red[tid >> 5] = lsum;
      __syncthreads();
      if (tid == 0) {
        float tot = 0.f;
        for (int i = 0; i < ST_THREADS / 32; ++i) tot += red[i];
        s.sums[frame * s.C + c] = tot;
      }
    }
  }
}

// Fast path of the plane stencil for 64x64 and 32x32 planes: float4 loads with the next
// step's plane prefetched into registers, the temporal history in registers, the spatial
// conv from a zero-haloed shared tile, per-step sums reduced once at the end.
// NP = float4 groups per thread = H*W / 1024.
template <int KSP, int KT, int NP>
__global__ void __launch_bounds__(ST_THREADS) plane_stencil_fast_kernel(const StencilArgs s) {
  extern __shared__ __align__(16) float sm[];
  const int H = s.H, W = s.W, HW = H * W;
  const int RS = W + 8;                              // tile row stride (4-float pad each side)
  float* tile = sm;                                  // [(H+2)][RS], used when KSP > 0
  float* red = sm + (KSP > 0 ? (H + 2) * RS : 0);    // [T][8] per-warp partial sums
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / s.C, c = blockIdx.x % s.C;
  constexpr int NHIST = KT > 0 ? KT - 1 : 0;

  float wsp[KSP * KSP > 0 ? KSP * KSP : 1];
  if (KSP > 0) {
#pragma unroll
    for (int i = 0; i < KSP * KSP; ++i) wsp[i] = s.wsp[(size_t)i * s.C + c];
  }
  const float bsp = KSP > 0 ? s.bsp[c] : 0.f;
  float wt[KT > 0 ? KT : 1];
  if (KT > 0) {
#pragma unroll
    for (int j = 0; j < KT; ++j) wt[j] = s.wt[(size_t)j * s.C + c];
  }
  const float btv = KT > 0 ? s.bt[c] : 0.f;
  if (KSP > 0) {
    for (int i = tid; i < (H + 2) * RS; i += ST_THREADS) tile[i] = 0.f;
  }
  float4 hist[NP][NHIST > 0 ? NHIST : 1];
#pragma unroll
  for (int j = 0; j < NP; ++j)
#pragma unroll
    for (int k = 0; k < NHIST; ++k) hist[j][k] = make_float4(0.f, 0.f, 0.f, 0.f);

  const size_t pstride = (size_t)s.planes_per_frame * HW;       // plane of the next frame
  float* p0 = s.buf + ((size_t)(b * s.T) * s.planes_per_frame + s.plane0 + c) * HW;
  float4 cur[NP], nxt[NP];
  int toff[NP];                    // tile offset of the thread's group j (interior origin)
  const int gpr = W >> 2;          // float4 groups per image row; lanes are consecutive groups
  bool left_edge[NP], right_edge[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int g4 = tid + j * ST_THREADS;
    cur[j] = reinterpret_cast<const float4*>(p0)[g4];
    const int h = g4 / gpr, gc = g4 - h * gpr;
    toff[j] = (h + 1) * RS + 4 + gc * 4;
    left_edge[j] = gc == 0 || lane == 0;
    right_edge[j] = gc == gpr - 1 || lane == 31;
  }
  __syncthreads();

  for (int t = 0; t < s.T; ++t) {
    float* p = p0 + (size_t)t * pstride;
    if (t + 1 < s.T) {
#pragma unroll
      for (int j = 0; j < NP; ++j)
        nxt[j] = reinterpret_cast<const float4*>(p + pstride)[tid + j * ST_THREADS];
    }
    if (KSP > 0) {
#pragma unroll
      for (int j = 0; j < NP; ++j) *reinterpret_cast<float4*>(tile + toff[j]) = cur[j];
      __syncthreads();
    }
    float lsum = 0.f;
    float4 outv[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      const int g4 = tid + j * ST_THREADS;
      float4 v = cur[j];
      if (KSP == 3) {
        // 3x3: the row's float4 from the tile, its left / right neighbours from the adjacent
        // lanes (adjacent float4 groups of the same image row) or from the zero halo
        float a0 = bsp, a1 = bsp, a2 = bsp, a3 = bsp;
#pragma unroll
        for (int di = 0; di < 3; ++di) {
          const float* rp = tile + toff[j] + (di - 1) * RS;
          const float4 mid = *reinterpret_cast<const float4*>(rp);
          float lf = __shfl_up_sync(0xffffffffu, mid.w, 1);
          float rt = __shfl_down_sync(0xffffffffu, mid.x, 1);
          if (left_edge[j]) lf = rp[-1];
          if (right_edge[j]) rt = rp[4];
          const float w0 = wsp[di * 3], w1 = wsp[di * 3 + 1], w2 = wsp[di * 3 + 2];
          a0 = fmaf(w0, lf, a0);    a0 = fmaf(w1, mid.x, a0); a0 = fmaf(w2, mid.y, a0);
          a1 = fmaf(w0, mid.x, a1); a1 = fmaf(w1, mid.y, a1); a1 = fmaf(w2, mid.z, a1);
          a2 = fmaf(w0, mid.y, a2); a2 = fmaf(w1, mid.z, a2); a2 = fmaf(w2, mid.w, a2);
          a3 = fmaf(w0, mid.z, a3); a3 = fmaf(w1, mid.w, a3); a3 = fmaf(w2, rt, a3);
        }
        v = make_float4(a0, a1, a2, a3);
      } else if (KSP > 0) {
        constexpr int LO = (KSP - 1) / 2;
        float a0 = bsp, a1 = bsp, a2 = bsp, a3 = bsp;
#pragma unroll
        for (int di = 0; di < KSP; ++di) {
          const float* rp = tile + toff[j] + (di - LO) * RS;
          float win[4 + 2 * LO];
          const float4 mid = *reinterpret_cast<const float4*>(rp);
          win[LO] = mid.x; win[LO + 1] = mid.y; win[LO + 2] = mid.z; win[LO + 3] = mid.w;
#pragma unroll
          for (int e = 0; e < LO; ++e) { win[e] = rp[e - LO]; win[LO + 4 + e] = rp[4 + e]; }
#pragma unroll
          for (int dj = 0; dj < KSP; ++dj) {
            const float wv = wsp[di * KSP + dj];
            a0 = fmaf(wv, win[dj], a0); a1 = fmaf(wv, win[dj + 1], a1);
            a2 = fmaf(wv, win[dj + 2], a2); a3 = fmaf(wv, win[dj + 3], a3);
          }
        }
        v = make_float4(a0, a1, a2, a3);
      }
      float4 o = v;
      if (KT > 0) {
        o = make_float4(btv + wt[KT - 1] * v.x, btv + wt[KT - 1] * v.y, btv + wt[KT - 1] * v.z,
                        btv + wt[KT - 1] * v.w);
        // hist[j][k] holds s_{t-1-k}; tap index of s_{t-1-k} is KT-2-k
#pragma unroll
        for (int k = 0; k < NHIST; ++k) {
          const float wv = wt[KT - 2 - k];
          o.x = fmaf(wv, hist[j][k].x, o.x); o.y = fmaf(wv, hist[j][k].y, o.y);
          o.z = fmaf(wv, hist[j][k].z, o.z); o.w = fmaf(wv, hist[j][k].w, o.w);
        }
#pragma unroll
        for (int k = NHIST - 1; k > 0; --k) hist[j][k] = hist[j][k - 1];
        if (NHIST > 0) hist[j][0] = v;
      }
      if (s.act) { o.x = silu_f(o.x); o.y = silu_f(o.y); o.z = silu_f(o.z); o.w = silu_f(o.w); }
      if (s.post) {
        const float* pp = s.post + ((size_t)(b * s.T + t) * HW + (size_t)g4 * 4) * s.post_stride + s.post_off;
        o.x *= pp[0]; o.y *= pp[s.post_stride]; o.z *= pp[2 * s.post_stride]; o.w *= pp[3 * s.post_stride];
      }
      outv[j] = o;
      lsum += (o.x + o.y) + (o.z + o.w);
    }
    // stores after all shared-memory reads of this step (generic-pointer stores would otherwise
    // pin the following loads behind them)
#pragma unroll
    for (int j = 0; j < NP; ++j) reinterpret_cast<float4*>(p)[tid + j * ST_THREADS] = outv[j];
    if (s.sums) {
      for (int off = 16; off > 0; off >>= 1) lsum += __shfl_down_sync(0xffffffffu, lsum, off);
      if (lane == 0) red[t * 8 + warp] = lsum;
    }
    if (KSP > 0) __syncthreads();      // all conv reads done before the tile is overwritten
#pragma unroll
    for (int j = 0; j < NP; ++j) cur[j] = nxt[j];
  }
  if (s.sums) {
    __syncthreads();
    for (int t = tid; t < s.T; t += ST_THREADS) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += red[t * 8 + w];
      s.sums[(size_t)(b * s.T + t) * s.C + c] = tot;
    }
  }
}

template <int KSP, int KT, int NP>
static int launch_stencil_fast(const StencilArgs& s, cudaStream_t st) {
  const size_t smem = ((KSP > 0 ? (size_t)(s.H + 2) * (s.W + 8) : 0) + (size_t)s.T * 8) * sizeof(float);
  if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(plane_stencil_fast_kernel<KSP, KT, NP>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  plane_stencil_fast_kernel<KSP, KT, NP><<<s.B * s.C, ST_THREADS, smem, st>>>(s);
  return check_launch();
}

template <int NP>
static int dispatch_stencil_fast(const StencilArgs& s, cudaStream_t st, bool* handled) {
  *handled = true;
  if (s.ksp == 3 && s.kt == 4) return launch_stencil_fast<3, 4, NP>(s, st);
  if (s.ksp == 0 && s.kt == 4) return launch_stencil_fast<0, 4, NP>(s, st);
  if (s.ksp == 3 && s.kt == 0) return launch_stencil_fast<3, 0, NP>(s, st);
  if (s.ksp == 0 && s.kt == 0) return launch_stencil_fast<0, 0, NP>(s, st);
  *handled = false;
  return CSSM_OK;
}

int launch_plane_stencil(const StencilArgs& s, cudaStream_t st) {
  if (s.ksp > 7 || s.kt > 8) return CSSM_ERR_UNSUPPORTED;
  if (s.W % 4 == 0 && (s.H * s.W == 4096 || s.H * s.W == 1024) &&
      (reinterpret_cast<uintptr_t>(s.buf) & 15u) == 0) {
    bool handled = false;
    const int rc = s.H * s.W == 4096 ? dispatch_stencil_fast<4>(s, st, &handled)
                                     : dispatch_stencil_fast<1>(s, st, &handled);
    if (handled) return rc;
  }
  const int nh = s.kt > 0 ? s.kt - 1 : 0;
  const size_t smem = (size_t)(1 + nh) * s.H * s.W * sizeof(float);
  if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  auto go = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    kern<<<s.B * s.C, ST_THREADS, smem, st>>>(s);
    return check_launch();
  };
  if (s.ksp == 3 && s.kt == 4) return go(plane_stencil_kernel<3, 4>);
  if (s.ksp == 0 && s.kt == 4) return go(plane_stencil_kernel<0, 4>);
  if (s.ksp == 3 && s.kt == 0) return go(plane_stencil_kernel<3, 0>);
  if (s.ksp == 0 && s.kt == 0) return go(plane_stencil_kernel<0, 0>);
  return go(plane_stencil_kernel<-1, -1>);
}

// ------------------------------------------- temporal conv on q, k, v (GDN) ----
// Causal depthwise temporal conv (KT taps) + SiLU + optional per-pixel input gate on the 3C planar
// planes of q, k and v in ONE elementwise launch: a thread owns four consecutive pixels of one
// plane and walks t with the KT-1 previous raw values in registers and the next frame's load in
// flight, so every plane is read once and written once at full occupancy.
template <int KT>
__global__ void __launch_bounds__(256) qkv_temporal_conv_kernel(const QkvTconvArgs a) {
  const int HW4 = a.HW >> 2;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long total = (long long)a.B * 3 * a.C * HW4;
  if (gid >= total) return;
  const int g4 = (int)(gid % HW4);
  const int p = (int)((gid / HW4) % (3 * a.C));
  const int b = (int)(gid / ((long long)HW4 * 3 * a.C));
  const int grp = p / a.C, c = p - grp * a.C;
  const float* wtp = grp == 0 ? a.wt[0] : grp == 1 ? a.wt[1] : a.wt[2];
  const float* btp = grp == 0 ? a.bt[0] : grp == 1 ? a.bt[1] : a.bt[2];
  float w[KT];
#pragma unroll
  for (int j = 0; j < KT; ++j) w[j] = wtp[(size_t)j * a.C + c];
  const float bias = btp[c];
  const int poff = grp - 1;                                   // k: B_k, v: B_v, q: none
  const bool gated = a.bkv != nullptr && grp > 0;
  float4 hist[KT - 1];
#pragma unroll
  for (int k = 0; k < KT - 1; ++k) hist[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t fstride = (size_t)3 * a.C * HW4;               // float4 units between frames
  float4* ptr = reinterpret_cast<float4*>(a.buf) + ((size_t)b * a.T * 3 * a.C + p) * HW4 + g4;
  float4 cur = *ptr;
  for (int t = 0; t < a.T; ++t) {
    float4 nxt = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t + 1 < a.T) nxt = ptr[fstride];
    // out[t] = bias + sum_j w[j] * s[t - (KT-1) + j]; hist[k] holds s[t - (KT-1) + k]
    float4 o = make_float4(fmaf(w[KT - 1], cur.x, bias), fmaf(w[KT - 1], cur.y, bias),
                           fmaf(w[KT - 1], cur.z, bias), fmaf(w[KT - 1], cur.w, bias));
#pragma unroll
    for (int k = 0; k < KT - 1; ++k) {
      o.x = fmaf(w[k], hist[k].x, o.x); o.y = fmaf(w[k], hist[k].y, o.y);
      o.z = fmaf(w[k], hist[k].z, o.z); o.w = fmaf(w[k], hist[k].w, o.w);
    }
#pragma unroll
    for (int k = 0; k + 1 < KT - 1; ++k) hist[k] = hist[k + 1];
    if (KT > 1) hist[KT - 2] = cur;
    o = make_float4(silu_f(o.x), silu_f(o.y), silu_f(o.z), silu_f(o.w));
    if (gated) {
      const float4* gp = reinterpret_cast<const float4*>(a.bkv + ((size_t)(b * a.T + t) * a.HW + 4 * g4));
      const float4 g0 = __ldg(gp), g1 = __ldg(gp + 1);        // {Bk,Bv} of pixels 0,1 and 2,3
      o.x *= poff ? g0.y : g0.x; o.y *= poff ? g0.w : g0.z;
      o.z *= poff ? g1.y : g1.x; o.w *= poff ? g1.w : g1.z;
    }
    *ptr = o;
    ptr += fstride;
    cur = nxt;
  }
}

int launch_qkv_temporal_conv(const QkvTconvArgs& a, cudaStream_t st) {
  if (a.HW % 4 != 0 || a.kt < 1) return CSSM_ERR_UNSUPPORTED;
  const long long total = (long long)a.B * 3 * a.C * (a.HW >> 2);
  const unsigned grid = (unsigned)((total + 255) / 256);
  switch (a.kt) {
    case 2: qkv_temporal_conv_kernel<2><<<grid, 256, 0, st>>>(a); break;
    case 3: qkv_temporal_conv_kernel<3><<<grid, 256, 0, st>>>(a); break;
    case 4: qkv_temporal_conv_kernel<4><<<grid, 256, 0, st>>>(a); break;
    default: return CSSM_ERR_UNSUPPORTED;
  }
  return check_launch();
}

// ----------------------------------------------------------- gated gate maps ----
// One CTA per (b,t).  ctx = ctx_sum / (H*W).  Writes, per bin, the float4
// {exp(-D), (D+1e-8)*Bg, Cg/(H*W), 1e-7*(D+1e-8)} at bin_index(path, kh, kw).

__device__ __forceinline__ float gate_act(float x, int act) {
  if (act == CSSM_ACT_SIGMOID2) return 2.0f / (1.0f + expf(-x));
  if (act == CSSM_ACT_EXP_CLIP) return expf(fminf(fmaxf(x, -4.f), 2.f));
  return x > 20.f ? x : log1pf(expf(x));
}

__global__ void __launch_bounds__(256) gated_gates_kernel(const GatedGateArgs g) {
  extern __shared__ float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf;
  float* ctx = sh;                 // [C]
  float* vec = sh + g.C;           // factored: 3 x (H + Wf)
  const int bt = blockIdx.x, tid = threadIdx.x;
  const float inv = 1.0f / (float)(g.H * g.W);
  for (int i = tid; i < g.C; i += blockDim.x) ctx[i] = g.ctx_sum[(size_t)bt * g.C + i] * inv;
  __syncthreads();
  if (g.gate_type == CSSM_GATE_FACTORED) {
    const int per = g.H + Wf;
    for (int o = tid; o < 3 * per; o += blockDim.x) {
      const int gi = o / per, r = o % per;
      const bool isw = r >= g.H;
      const int col = isw ? r - g.H : r, ncol = isw ? Wf : g.H;
      const float* kk = g.gk[2 * gi + (isw ? 1 : 0)];
      float acc = g.gb[2 * gi + (isw ? 1 : 0)][col];
      for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * ncol + col], acc);
      vec[o] = acc;
    }
    __syncthreads();
  }
  // the bins of a frame are split over gridDim.y CTAs (few frames, many bins: dense gates)
  const int per_cta = (NB + gridDim.y - 1) / gridDim.y;
  const int bin_end = min(NB, (int)(blockIdx.y + 1) * per_cta);
  for (int bin = blockIdx.y * per_cta + tid; bin < bin_end; bin += blockDim.x) {
    const int kh = bin / Wf, kw = bin % Wf;
    float r[3];
    if (g.gate_type == CSSM_GATE_FACTORED) {
      const int per = g.H + Wf;
#pragma unroll
      for (int gi = 0; gi < 3; ++gi) r[gi] = vec[gi * per + kh] * vec[gi * per + g.H + kw];
    } else {
#pragma unroll
      for (int gi = 0; gi < 3; ++gi) {
        float acc = g.gb[gi][bin];
        const float* kk = g.gk[gi];
        for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * NB + bin], acc);
        r[gi] = acc;
      }
    }
    const float D = gate_act(r[0], g.act);
    float4 o;
    o.x = expf(-D);
    o.y = (D + 1e-8f) * r[1];
    o.z = r[2] * inv;
    o.w = 1e-7f * (D + 1e-8f);
    g.maps[(size_t)bt * NB + bin_index(g.path, kh, kw, g.H, Wf)] = o;
  }
}

// Factored gates of many frames with small planes (the CSSM-SHViT stages: hundreds of frames of
// 14x14 / 7x7).  A CTA takes GB_FR frames.  It first copies the six gate matrices (C x H and C x Wf
// each, at most ~100 KB) to shared memory with every thread's 16-byte loads all in flight at once (a
// walk through them with a few loads per thread in flight is a chain of cold misses: 31 us); then a
// thread computes whole gate-vector entries (one dot product over the C channels) and the bins are
// written.
constexpr int GB_FR = 4;
__global__ void __launch_bounds__(256) gated_gates_batched_kernel(const GatedGateArgs g) {
  extern __shared__ __align__(16) float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf, per = g.H + Wf;
  const int nH = g.C * g.H, nW = g.C * Wf;           // floats per matrix (multiples of 4: C % 4 == 0)
  float* wsm = sh;                         // six matrices as they lie in memory: [gate][H part | Wf part]
  float* ctx = wsm + 3 * (nH + nW);        // [GB_FR][C]
  float* vec = ctx + GB_FR * g.C;          // [GB_FR][3][per]: the H then the Wf entries of each gate
  const int tid = threadIdx.x;
  const int f0 = blockIdx.x * GB_FR;
  const int nf = g.BT - f0 < GB_FR ? g.BT - f0 : GB_FR;
  const float inv = 1.0f / (float)(g.H * g.W);
  {
    const int q4H = nH / 4, q4W = nW / 4, tot4 = 3 * (q4H + q4W);
    for (int i0 = tid; i0 < tot4; i0 += 16 * 256) {
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = i0 + u * 256;
        if (i < tot4) {
          const int gi = i / (q4H + q4W), r = i - gi * (q4H + q4W);
          v[u] = r < q4H ? __ldg(reinterpret_cast<const float4*>(g.gk[2 * gi]) + r)
                         : __ldg(reinterpret_cast<const float4*>(g.gk[2 * gi + 1]) + (r - q4H));
        }
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = i0 + u * 256;
        if (i < tot4) reinterpret_cast<float4*>(wsm)[i] = v[u];
      }
    }
  }
  for (int i = tid; i < nf * g.C; i += blockDim.x) ctx[i] = g.ctx_sum[(size_t)f0 * g.C + i] * inv;
  __syncthreads();
  for (int idx = tid; idx < nf * 3 * per; idx += blockDim.x) {
    const int f = idx / (3 * per), o = idx - f * 3 * per;
    const int gi = o / per, col = o - gi * per;
    const bool wpart = col >= g.H;
    const int cc = wpart ? col - g.H : col, ncol = wpart ? Wf : g.H;
    const float* src = wsm + gi * (nH + nW) + (wpart ? nH : 0) + cc;
    const float* cx = ctx + f * g.C;
    float acc[4] = {g.gb[2 * gi + (wpart ? 1 : 0)][cc], 0.f, 0.f, 0.f};
    int c = 0;
    for (; c + 4 <= g.C; c += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = fmaf(cx[c + u], src[(c + u) * ncol], acc[u]);
    }
    for (; c < g.C; ++c) acc[0] = fmaf(cx[c], src[c * ncol], acc[0]);
    vec[idx] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  }
  __syncthreads();
  for (int idx = tid; idx < nf * NB; idx += blockDim.x) {
    const int f = idx / NB, bin = idx - f * NB;
    const int kh = bin / Wf, kw = bin - kh * Wf;
    const float* v = vec + f * 3 * per;
    float r[3];
#pragma unroll
    for (int gi = 0; gi < 3; ++gi) r[gi] = v[gi * per + kh] * v[gi * per + g.H + kw];
    const float D = gate_act(r[0], g.act);
    float4 o;
    o.x = expf(-D);
    o.y = (D + 1e-8f) * r[1];
    o.z = r[2] * inv;
    o.w = 1e-7f * (D + 1e-8f);
    g.maps[(size_t)(f0 + f) * NB + bin_index(g.path, kh, kw, g.H, Wf)] = o;
  }
}

int launch_gated_gates(const GatedGateArgs& g, cudaStream_t st) {
  const int Wf = g.W / 2 + 1;
  {
    const size_t per = (size_t)g.H + Wf;
    const size_t bsm = ((size_t)3 * g.C * per + (size_t)GB_FR * (g.C + 3 * per)) * sizeof(float);
    bool al = g.C % 4 == 0;
    for (int i = 0; i < 6; ++i) al = al && aligned16(g.gk[i]);
    if (g.gate_type == CSSM_GATE_FACTORED && g.BT >= 64 && g.H * Wf <= 256 && bsm <= 160 * 1024 && al) {
      cudaError_t e = cudaFuncSetAttribute(gated_gates_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)bsm);
      if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
      gated_gates_batched_kernel<<<(g.BT + GB_FR - 1) / GB_FR, 256, bsm, st>>>(g);
      return check_launch();
    }
  }
  const size_t smem = (size_t)(g.C + 3 * (g.H + Wf)) * sizeof(float);
  // enough CTAs to cover the GPU when there are few frames: up to one CTA per 256 bins
  const int NB = g.H * Wf;
  int chunks = 1;
  if (g.BT < 296) {
    chunks = (296 + g.BT - 1) / g.BT;
    const int maxc = (NB + 255) / 256;
    if (chunks > maxc) chunks = maxc;
  }
  gated_gates_kernel<<<dim3(g.BT, chunks), 256, smem, st>>>(g);
  return check_launch();
}

}  // namespace cssm
