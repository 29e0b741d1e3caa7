// Fused spectral kernels of the gated block: rfft2 -> gated complex recurrence over T with
// the state on chip -> irfft2 -> * silu(z) (in_proj already stored the z planes through SiLU).
// One CTA per (batch, channel) pair.
#include <cuda.h>
#include <string.h>
#include "r64.cuh"
#include "kernels.cuh"
#include "tc05.cuh"

namespace cssm {

// ============================================================== 64 x 64 planes ====
// 288 threads; thread roles and shared-memory layout are those of r64.cuh.  The lane keeps the
// state of its 8 bins (kh = a + 8q of column grp) in registers for all T steps.
// The x_main plane of step t+1 and the (SiLU'd) z plane of step t+1 are staged in shared memory
// by TMA tensor copies (one per plane, issued by a lane of the otherwise idle ninth warp right
// after the first barrier of step t) and land while step t computes; gate maps and K_hat are
// loaded at the top of the column phase.  The copy's 68-wide box over the 64-wide rows pads every
// row to 272 bytes (the four out-of-bounds columns arrive as zeros), which makes the row passes'
// reads bank-conflict free.
// A bounded mbarrier wait that expires records a code in g_spec_error (read it with
// cssm_device_error) and the whole CTA leaves its step loop at the next barrier without storing
// anything more.
constexpr int R64_THREADS = R64_NT;
constexpr int R64_PLANE_F = 64 * 68;
constexpr int R64_SMEM_BYTES = (R64_EX_CF + R64_ZR_CF + R64_GB_CF) * 8 + 3 * R64_PLANE_F * 4 + 128;

__device__ int g_spec_error = 0;
int launch_gated_spectral_r32(float* xz, const cf* khat, const float* gates, int B, int T, int C,
                              int last_only, int nogate, cudaStream_t st, const float* dchan);

// LAST: only the last step's output plane is produced (compile-time, so that the all-frames
// kernel carries none of the branches).
// MODE 0: gated block (gate maps, output times the silu(z) plane).  MODE 1: the ungated recurrence
// S_t = K_hat S_{t-1} + X_hat_t of NoGateCSSM (no gate maps, no z plane).  MODE 2: gate maps but no
// z plane (the single-state AdditiveCSSM).  MODE 3: MODE 2 with a per-(frame, channel) decay dchan[frame, c]
// on top of the maps (the additive block's per-channel gates).
template <bool LAST, int MODE>
__global__ void __launch_bounds__(R64_THREADS, 2)
gated_spectral_r64(float* __restrict__ xz, const cf* __restrict__ khat,
                   const float4* __restrict__ gates, int T, int C,
                   const __grid_constant__ CUtensorMap pmap, const float* __restrict__ dchan) {
  constexpr int last_only = LAST ? 1 : 0;
  constexpr int PRS = 68;                                     // floats per staged row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // TMA tensor copies need a 128-byte aligned destination; dynamic shared memory is only
  // guaranteed 16-byte aligned, so the base is rounded up (the launch adds 128 bytes)
  unsigned char* smem_al = smem_raw + ((128u - (tc::smem_u32(smem_raw) & 127u)) & 127u);
  cf* EX = reinterpret_cast<cf*>(smem_al);
  float* xbuf = reinterpret_cast<float*>(EX + R64_EX_CF + R64_ZR_CF + R64_GB_CF);
  constexpr int R64_PRS = PRS;
  float* zbuf = xbuf + R64_PLANE_F;                           // two buffers
  __shared__ __align__(8) uint64_t bars[3];                   // x, z[0], z[1]
  __shared__ int s_bad;                                       // a bounded wait expired
  R64Ctx c;
  r64_init(c, EX, EX + R64_EX_CF, EX + R64_EX_CF + R64_ZR_CF);

  const int b = blockIdx.x / C, ch = blockIdx.x % C;
  constexpr int HW = 64 * 64;
  const cf* khp = khat + (size_t)ch * (64 * 33) + (c.grp << 3) + c.a;
  const float* x0 = xz + ((size_t)(b * T) * 2 * C + ch) * HW;          // x_main plane of step 0
  const size_t fstride = (size_t)2 * C * HW;                            // next step's plane

  if (threadIdx.x == 0) {
    tc::mbar_init(&bars[0], 1); tc::mbar_init(&bars[1], 1); tc::mbar_init(&bars[2], 1);
    tc::fence_mbar_init();
    s_bad = 0;
  }
  __syncthreads();
  // stage step `tl`: x_main plane into xbuf (if want_x) and z plane into zbuf[tl & 1]
  auto stage = [&](int tl, bool want_x) {
    if (c.warp != 8) return;
    const bool want_z = MODE == 0 && (!last_only || tl == T - 1);
    tc::fence_proxy_async();             // earlier generic reads of the buffers come first
    uint64_t* bz = &bars[1 + (tl & 1)];
    if (c.lane == 0) {
      if (want_x) tc::mbar_expect_tx(&bars[0], 64 * PRS * 4);
      if (want_z) tc::mbar_expect_tx(bz, 64 * PRS * 4);
    }
    __syncwarp();
    const float* xs = x0 + (size_t)tl * fstride;
    const float* zs = xs + (size_t)C * HW;
    float* zd = zbuf + (tl & 1) * R64_PLANE_F;
    // one tensor copy per plane: the 68-wide box reads 4 columns past the 64-wide rows, which
    // are out of bounds for the map and arrive as zeros, so the rows land 272 bytes apart
    if (c.lane == 0) {
      const int row0 = (int)((xs - xz) >> 6);           // first image row of the plane
      if (want_x) tc::tma_load_2d(xbuf, &pmap, 0, row0, &bars[0]);
      if (want_z) tc::tma_load_2d(zd, &pmap, 0, row0 + C * 64, bz);
    }
  };
  stage(0, true);

  cf hst[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) hst[q] = mk(0.f, 0.f);
  const int roff = (2 * c.grp) * 64 + c.a;              // global offset of the lane's row pair
  const int soff = (2 * c.grp) * R64_PRS + c.a;         // same inside a staged plane

  for (int t = 0; t < T; ++t) {
    const size_t frame = (size_t)(b * T + t);
    float* xp = xz + (frame * 2 * C + ch) * HW;
    const bool emit = !last_only || t == T - 1;       // same for the whole CTA

    // ---- forward rows (from the staged plane) ----
    if (c.row_on) {
      if (!tc::mbar_wait(&bars[0], t & 1)) { atomicExch(&g_spec_error, 1); s_bad = 1; }
      cf v[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) v[m] = mk(xbuf[soff + 8 * m], xbuf[soff + R64_PRS + 8 * m]);
      fft64_lane8<false>(v, c.tw, c.exg, c.a);
#pragma unroll
      for (int k2 = 0; k2 < 8; ++k2) c.ZR[c.grp * R64_ZRS + c.a + 8 * k2] = v[k2];
    }
    __syncthreads();
    if (s_bad) break;                                 // same for the whole CTA (read after the barrier)
    if (t + 1 < T) stage(t + 1, true);

    // ---- forward columns, recurrence, inverse columns ----
    if (c.col_warp) {
      float4 g[8];
      cf kh[8];
      const float4* gp = gates + frame * (64 * 33) + (c.grp << 3) + c.a;
      // MODE 3: the decay of this (frame, channel) multiplies the map's decay entry
      const float dc = MODE == 3 ? __ldg(dchan + frame * C + ch) : 1.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        // {exp(-D), (D+1e-8)B, C/(HW), 1e-7(D+1e-8)}
        if (MODE != 1) g[q] = c.col_on ? __ldg(gp + q * (33 * 8)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE == 3) g[q].x *= dc;
        kh[q] = c.col_on ? khp[q * (33 * 8)] : mk(0.f, 0.f);
      }
      cf v[8];
      r64_col_fwd(c, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (MODE == 1) {
          cf h = cmul(kh[q], hst[q]);
          h.x += v[q].x; h.y += v[q].y;
          hst[q] = h;
          v[q] = mk(h.x * (1.0f / HW), h.y * (1.0f / HW));
        } else {
          const cf A = mk(kh[q].x * g[q].x, kh[q].y * g[q].x);
          cf U = mk(g[q].y * v[q].x, g[q].y * v[q].y);
          if (U.x * U.x + U.y * U.y < g[q].w * g[q].w) U = mk(g[q].w, 0.f);
          cf h = cmul(A, hst[q]);
          h.x += U.x; h.y += U.y;
          hst[q] = h;
          v[q] = mk(g[q].z * h.x, g[q].z * h.y);
        }
      }
      if (emit) r64_col_inv(c, v);
    }
    __syncthreads();

    // ---- inverse rows, * staged silu(z), store ----
    if (c.row_on && emit) {
      cf v[8];
      r64_row_inv(c, v);
      float* y0 = xp + roff;
      if (MODE == 0) {
        // in last-only mode the z barrier of this slot completes exactly once (phase 0)
        if (!tc::mbar_wait(&bars[1 + (t & 1)], last_only ? 0 : (t >> 1) & 1)) {
          atomicExch(&g_spec_error, 2); s_bad = 1;
          continue;                 // no store; the CTA leaves at the next step's first barrier
        }
        const float* zs = zbuf + (t & 1) * R64_PLANE_F + soff;
        // finish all products before the first store: the stores go through a generic pointer,
        // so shared-memory loads placed between them could not be hoisted
#pragma unroll
        for (int n1 = 0; n1 < 8; ++n1) v[n1] = mk(v[n1].x * zs[8 * n1], v[n1].y * zs[R64_PRS + 8 * n1]);
      }
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1) {
        y0[8 * n1] = v[n1].x;
        y0[64 + 8 * n1] = v[n1].y;
      }
    }
    // No barrier needed here: the next iteration writes EX (warp-private) and ZR (last read
    // before the second barrier above); GB is next written after the next first barrier; xbuf
    // and zbuf[(t+1)&1] are refilled only after the next first barrier.
  }
  // error path only: give copies that may still be in flight a bounded time (~1 ms) to land before
  // the CTA's shared memory is released
  if (s_bad)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
}

int read_spec_error(int* out, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_spec_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_spec_error, &zero, sizeof(int));
  }
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

// ================================================================ generic planes ====
// Any H, W: direct DFTs with twiddle tables in shared memory.  Slow (O(N) per output)
// but exact in structure; used for plane sizes without a radix kernel and as an
// independent CUDA cross-check of the radix kernel in the tests.
constexpr int GEN_THREADS = 256;

__global__ void __launch_bounds__(GEN_THREADS)
gated_spectral_generic(float* __restrict__ xz, const cf* __restrict__ khat,
                       const float4* __restrict__ gates, int T, int C, int H, int W, int last_only,
                       int nog, const float* __restrict__ dchan) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf;
  float* xs = reinterpret_cast<float*>(smem_raw);              // [H][W]
  cf* twW = reinterpret_cast<cf*>(xs + ((HW + 1) & ~1));       // [W]  e^{-2 pi i k/W}
  cf* twH = twW + W;                                           // [H]
  cf* Rb = twH + H;                                            // [H][Wf]
  cf* Fb = Rb + NB;                                            // [H][Wf]
  cf* St = Fb + NB;                                            // [H][Wf] state

  const int tid = threadIdx.x;
  const int b = blockIdx.x / C, c = blockIdx.x % C;
  for (int i = tid; i < W; i += GEN_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)W, &s, &co); twW[i] = mk(co, s);
  }
  for (int i = tid; i < H; i += GEN_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)H, &s, &co); twH[i] = mk(co, s);
  }
  for (int i = tid; i < NB; i += GEN_THREADS) St[i] = mk(0.f, 0.f);
  const cf* khc = khat + (size_t)c * NB;

  for (int t = 0; t < T; ++t) {
    const size_t frame = (size_t)(b * T + t);
    float* xp = xz + (frame * 2 * C + c) * HW;
    const float* zp = xz + (frame * 2 * C + C + c) * HW;
    __syncthreads();
    for (int i = tid; i < HW; i += GEN_THREADS) xs[i] = xp[i];
    __syncthreads();
    // rows: R[h][kw] = sum_w x[h][w] e^{-2 pi i w kw / W}
    for (int o = tid; o < NB; o += GEN_THREADS) {
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
    // columns + recurrence
    const float4* gp = gates + frame * NB;
    for (int o = tid; o < NB; o += GEN_THREADS) {
      const int kh = o / Wf, kw = o % Wf;
      float ax = 0.f, ay = 0.f;
      int idx = 0;
      for (int h = 0; h < H; ++h) {
        const cf e = twH[idx];
        const cf r = Rb[h * Wf + kw];
        ax += r.x * e.x - r.y * e.y; ay += r.x * e.y + r.y * e.x;
        idx += kh; if (idx >= H) idx -= H;
      }
      // ungated mode: A = K_hat, U = X_hat, output scale 1/(H*W), no floor
      float4 g = nog == 1 ? make_float4(1.f, 1.f, 1.0f / (float)HW, 0.f) : gp[o];
      if (nog == 3) g.x *= __ldg(dchan + frame * C + c);
      const cf k = khc[o];
      cf A = mk(k.x * g.x, k.y * g.x);
      cf U = mk(g.y * ax, g.y * ay);
      if (U.x * U.x + U.y * U.y < g.w * g.w) U = mk(g.w, 0.f);
      cf hs = cmul(A, St[o]);
      hs.x += U.x; hs.y += U.y;
      St[o] = hs;
      Fb[o] = mk(g.z * hs.x, g.z * hs.y);
    }
    if (last_only && t != T - 1) continue;        // uniform: the next step starts with a barrier
    __syncthreads();
    // inverse columns: R[h][kw] = sum_kh F[kh][kw] e^{+2 pi i h kh / H}
    for (int o = tid; o < NB; o += GEN_THREADS) {
      const int h = o / Wf, kw = o % Wf;
      float ax = 0.f, ay = 0.f;
      int idx = 0;
      for (int kh = 0; kh < H; ++kh) {
        const cf e = twH[idx];          // conj -> e^{+}
        const cf f = Fb[kh * Wf + kw];
        ax += f.x * e.x + f.y * e.y; ay += f.y * e.x - f.x * e.y;
        idx += h; if (idx >= H) idx -= H;
      }
      Rb[o] = mk(ax, ay);
    }
    __syncthreads();
    // inverse rows, C2R: imaginary parts of column 0 (and W/2 for even W) are ignored
    const int kmax = (W - 1) / 2;
    for (int o = tid; o < HW; o += GEN_THREADS) {
      const int h = o / W, w = o % W;
      const cf* r = Rb + h * Wf;
      float acc = r[0].x;
      if ((W & 1) == 0) acc += (w & 1) ? -r[W / 2].x : r[W / 2].x;
      int idx = 0;
      float s2 = 0.f;
      for (int k = 1; k <= kmax; ++k) {
        idx += w; if (idx >= W) idx -= W;
        const cf e = twW[idx];          // e^{-i th}: cos = e.x, sin = -e.y
        s2 += r[k].x * e.x + r[k].y * e.y;
      }
      acc += 2.f * s2;
      xp[o] = nog != 0 ? acc : acc * zp[o];
    }
  }
}

// ================================================================ small planes ====
// Planes of at most 16 x 16 pixels (the 14 x 14 and 7 x 7 stages of the SHViT backbone): one
// WARP per (batch, channel) plane, eight planes in flight per CTA, CTAs loop over the planes.
// Same direct-DFT arithmetic as the generic kernel, synchronised with __syncwarp() only, and the
// twiddle tables are built once per CTA instead of once per plane.
constexpr int SMALL_WARPS = 8, SMALL_MAX_HW = 256;

__global__ void __launch_bounds__(SMALL_WARPS * 32)
gated_spectral_small(float* __restrict__ xz, const cf* __restrict__ khat,
                     const float4* __restrict__ gates, int nplanes, int T, int C, int H, int W,
                     int last_only, int nog, const float* __restrict__ dchan) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  cf* twW = reinterpret_cast<cf*>(smem_raw);                   // [W]  e^{-2 pi i k/W}
  cf* twH = twW + W;                                           // [H]
  const int per_warp = ((HW + 1) & ~1) / 2 + 3 * NB;           // in cf units: xs, Rb, Fb, St
  cf* mine = twH + H + (size_t)warp * per_warp;
  float* xs = reinterpret_cast<float*>(mine);                  // [H][W]
  cf* Rb = mine + ((HW + 1) & ~1) / 2;                         // [H][Wf]
  cf* Fb = Rb + NB;
  cf* St = Fb + NB;
  for (int i = threadIdx.x; i < W; i += SMALL_WARPS * 32) {
    float s, co; sincospif(-2.0f * (float)i / (float)W, &s, &co); twW[i] = mk(co, s);
  }
  for (int i = threadIdx.x; i < H; i += SMALL_WARPS * 32) {
    float s, co; sincospif(-2.0f * (float)i / (float)H, &s, &co); twH[i] = mk(co, s);
  }
  __syncthreads();
  const float invHW = 1.0f / (float)HW;
  const int kmax = (W - 1) / 2;
  for (int plane = blockIdx.x * SMALL_WARPS + warp; plane < nplanes; plane += gridDim.x * SMALL_WARPS) {
    const int b = plane / C, c = plane % C;
    const cf* khc = khat + (size_t)c * NB;
    for (int i = lane; i < NB; i += 32) St[i] = mk(0.f, 0.f);
    for (int t = 0; t < T; ++t) {
      const size_t frame = (size_t)(b * T + t);
      float* xp = xz + (frame * 2 * C + c) * HW;
      const float* zp = xp + (size_t)C * HW;
      __syncwarp();
      for (int i = lane; i < HW; i += 32) xs[i] = xp[i];
      __syncwarp();
      for (int o = lane; o < NB; o += 32) {                    // rows
        const int h = o / Wf, kw = o - h * Wf;
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
      __syncwarp();
      const float4* gp = gates + frame * NB;
      for (int o = lane; o < NB; o += 32) {                    // columns + recurrence
        const int kh = o / Wf, kw = o - kh * Wf;
        float ax = 0.f, ay = 0.f;
        int idx = 0;
        for (int h = 0; h < H; ++h) {
          const cf e = twH[idx];
          const cf r = Rb[h * Wf + kw];
          ax += r.x * e.x - r.y * e.y; ay += r.x * e.y + r.y * e.x;
          idx += kh; if (idx >= H) idx -= H;
        }
        float4 g = nog == 1 ? make_float4(1.f, 1.f, invHW, 0.f) : __ldg(gp + o);
        if (nog == 3) g.x *= __ldg(dchan + frame * C + c);
        const cf k = khc[o];
        const cf A = mk(k.x * g.x, k.y * g.x);
        cf U = mk(g.y * ax, g.y * ay);
        if (U.x * U.x + U.y * U.y < g.w * g.w) U = mk(g.w, 0.f);
        cf hs = cmul(A, St[o]);
        hs.x += U.x; hs.y += U.y;
        St[o] = hs;
        Fb[o] = mk(g.z * hs.x, g.z * hs.y);
      }
      if (last_only && t != T - 1) continue;                   // same for the whole warp
      __syncwarp();
      for (int o = lane; o < NB; o += 32) {                    // inverse columns
        const int h = o / Wf, kw = o - h * Wf;
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
      __syncwarp();
      for (int o = lane; o < HW; o += 32) {                    // inverse rows (C2R), * silu(z)
        const int h = o / W, w = o - h * W;
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
        acc += 2.f * s2;
        xp[o] = nog != 0 ? acc : acc * zp[o];
      }
    }
  }
}

static size_t small_smem_bytes(int H, int W) {
  const size_t NB = (size_t)H * (W / 2 + 1), HW = (size_t)H * W;
  const size_t per_warp = ((HW + 1) & ~(size_t)1) / 2 + 3 * NB;
  return (W + H + SMALL_WARPS * per_warp) * sizeof(cf);
}

size_t generic_smem_bytes(int H, int W) {
  const int Wf = W / 2 + 1;
  size_t fl = ((size_t)H * W + 1) & ~(size_t)1;
  return fl * 4 + (size_t)(W + H + 3 * H * Wf) * sizeof(cf);
}

int launch_gated_spectral(const cssm_gated_desc& d, const cf* khat, const float* gates,
                          float* xz, int last_only, cudaStream_t st) {
  return launch_spectral(d.B, d.T, d.H, d.W, d.C, khat, gates, xz, last_only, 0, st);
}

int launch_spectral(int B, int T, int H, int W, int C, const cf* khat, const float* gates,
                    float* xz, int last_only, int nogate, cudaStream_t st, const float* dchan) {
  if ((nogate == 3) != (dchan != nullptr)) return CSSM_ERR_NULL;
  struct { int B, T, H, W, C; } d = {B, T, H, W, C};
  const SpectralPath path = spectral_path(d.H, d.W);
  const int grid = d.B * d.C;
  if (path == PATH_R32) return launch_gated_spectral_r32(xz, khat, gates, d.B, d.T, d.C, last_only, nogate, st, dchan);
  if (path == PATH_R64) {
    const size_t smem = R64_SMEM_BYTES;
    // tensor map over the planar buffer as rows of 64 floats; box 68 x 64 (see the kernel)
    CUtensorMap pmap;
    memset(&pmap, 0, sizeof(pmap));
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);
    static EncodeFn enc = []() -> EncodeFn {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
          q != cudaDriverEntryPointSuccess)
        return nullptr;
      return reinterpret_cast<EncodeFn>(p);
    }();
    const cuuint64_t dims[2] = {64, (cuuint64_t)d.B * d.T * 2 * d.C * 64};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {68, 64}, es[2] = {1, 1};
    if (enc == nullptr ||
        enc(&pmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, xz, dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return CSSM_ERR_CUDA;
    auto kern = last_only ? gated_spectral_r64<true, 0> : gated_spectral_r64<false, 0>;
    if (nogate == 1) kern = last_only ? gated_spectral_r64<true, 1> : gated_spectral_r64<false, 1>;
    else if (nogate == 2) kern = last_only ? gated_spectral_r64<true, 2> : gated_spectral_r64<false, 2>;
    else if (nogate == 3) kern = last_only ? gated_spectral_r64<true, 3> : gated_spectral_r64<false, 3>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    kern<<<grid, R64_THREADS, smem, st>>>(xz, khat, reinterpret_cast<const float4*>(gates), d.T,
                                          d.C, pmap, dchan);
  } else if (d.H * d.W <= SMALL_MAX_HW) {
    const size_t smem = small_smem_bytes(d.H, d.W);
    cudaError_t e = cudaFuncSetAttribute(gated_spectral_small,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    const int need = (grid + SMALL_WARPS - 1) / SMALL_WARPS;
    const int ctas = need < 148 * 6 ? need : 148 * 6;
    gated_spectral_small<<<ctas, SMALL_WARPS * 32, smem, st>>>(
        xz, khat, reinterpret_cast<const float4*>(gates), grid, d.T, d.C, d.H, d.W, last_only, nogate, dchan);
  } else {
    const size_t smem = generic_smem_bytes(d.H, d.W);
    if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(gated_spectral_generic,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    gated_spectral_generic<<<grid, GEN_THREADS, smem, st>>>(
        xz, khat, reinterpret_cast<const float4*>(gates), d.T, d.C, d.H, d.W, last_only, nogate, dchan);
  }
  return check_launch();
}

}  // namespace cssm
