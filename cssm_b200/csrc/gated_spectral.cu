// Fused spectral kernels of the gated block: rfft2 -> gated complex recurrence over T with
// the state on chip -> irfft2 -> * silu(z).  One CTA per (batch, channel) pair.
#include "fft.cuh"
#include "kernels.cuh"

namespace cssm {

// ============================================================== 64 x 64 planes ====
// 288 threads.  lane = sub + 4*a.  Row passes: warp w < 8 owns row pairs 4w + sub (two
// real rows packed into one complex 64-point FFT).  Column passes: warp w < 9 owns
// half-spectrum columns kw = 4w + sub (kw <= 32); the lane keeps the state of bins
// kh = a + 8b, b = 0..7, in registers for all T steps.
constexpr int R64_THREADS = 288;
constexpr int R64_ZR_STRIDE = 68;   // cf per packed row pair
constexpr int R64_GB_STRIDE = 34;   // cf per spatial row of the inverse column output
constexpr int R64_SMEM_CF = 36 * EX_GROUP_STRIDE + 32 * R64_ZR_STRIDE + 64 * R64_GB_STRIDE;

__global__ void __launch_bounds__(R64_THREADS, 2)
gated_spectral_r64(float* __restrict__ xz, const cf* __restrict__ khat,
                   const float4* __restrict__ gates, int T, int C) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZR = EX + 36 * EX_GROUP_STRIDE;
  cf* GB = ZR + 32 * R64_ZR_STRIDE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane & 3, a = lane >> 2;
  const int grp = warp * 4 + sub;            // row pair (row passes) / column (column passes)
  const bool row_on = warp < 8;
  // Column passes run on whole warps (the exchange inside the FFT synchronises the warp):
  // the three lanes groups of warp 8 beyond column 32 compute on in-bounds scratch and
  // only their global loads and shared-memory results are suppressed.
  const bool col_warp = warp < 9;
  const bool col_on = grp <= 32;
  cf* exg = EX + grp * EX_GROUP_STRIDE;

  const int b = blockIdx.x / C, c = blockIdx.x % C;
  constexpr int HW = 64 * 64;

  cf tw[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float s, co;
    sincospif(-(float)(a * k) / 32.0f, &s, &co);
    tw[k] = mk(co, s);
  }

  cf kh[8], hst[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    hst[q] = mk(0.f, 0.f);
    kh[q] = col_on ? khat[(size_t)c * (64 * 33) + ((q * 33 + grp) << 3) + a] : mk(0.f, 0.f);
  }

  for (int t = 0; t < T; ++t) {
    const size_t frame = (size_t)(b * T + t);
    float* xp = xz + (frame * 2 * C + c) * HW;
    const float* zp = xz + (frame * 2 * C + C + c) * HW;
    cf v[8];

    // ---- forward rows: two real rows as one complex FFT ----
    if (row_on) {
      const float* r0 = xp + (2 * grp) * 64 + a;
#pragma unroll
      for (int m = 0; m < 8; ++m) v[m] = mk(r0[8 * m], r0[64 + 8 * m]);
      fft64_lane8<false>(v, tw, exg, a);
#pragma unroll
      for (int k2 = 0; k2 < 8; ++k2) ZR[grp * R64_ZR_STRIDE + a + 8 * k2] = v[k2];
    }
    __syncthreads();

    // ---- forward columns, recurrence, inverse columns ----
    if (col_warp) {
      const int par = a & 1, ph = a >> 1;
      const int kneg = (64 - grp) & 63;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        cf z1 = ZR[(ph + 4 * m) * R64_ZR_STRIDE + grp];
        cf z2 = ZR[(ph + 4 * m) * R64_ZR_STRIDE + kneg];
        v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
                   : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
      }
      fft64_lane8<false>(v, tw, exg, a);
      const float4* gp = gates + frame * (64 * 33) + (grp << 3) + a;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        // {exp(-D), (D+1e-8)B, C/(HW), 1e-7(D+1e-8)}
        const float4 g = col_on ? gp[q * (33 * 8)] : make_float4(0.f, 0.f, 0.f, 0.f);
        cf A = mk(kh[q].x * g.x, kh[q].y * g.x);
        cf U = mk(g.y * v[q].x, g.y * v[q].y);
        if (U.x * U.x + U.y * U.y < g.w * g.w) U = mk(g.w, 0.f);
        cf h = cmul(A, hst[q]);
        h.x += U.x; h.y += U.y;
        hst[q] = h;
        v[q] = mk(g.z * h.x, g.z * h.y);
      }
      fft64_lane8<true>(v, tw, exg, a);
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1)
        if (col_on) GB[(a + 8 * n1) * R64_GB_STRIDE + grp] = v[n1];
    }
    __syncthreads();

    // ---- inverse rows (C2R, two rows per complex FFT), * silu(z), store ----
    if (row_on) {
      const cf* ge = GB + (2 * grp) * R64_GB_STRIDE;
      const cf* go = ge + R64_GB_STRIDE;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const int n = a + 8 * m;
        const int k = n <= 32 ? n : 64 - n;
        cf e = ge[k], o = go[k];
        if (m == 0 || m == 4) {           // n = a or a + 32: DC / Nyquist when a == 0
          if (a == 0) { e.y = 0.f; o.y = 0.f; }
        }
        v[m] = (n <= 32) ? mk(e.x - o.y, e.y + o.x) : mk(e.x + o.y, o.x - e.y);
      }
      fft64_lane8<true>(v, tw, exg, a);
      const float* z0 = zp + (2 * grp) * 64 + a;
      float* y0 = xp + (2 * grp) * 64 + a;
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1) {
        float ze = z0[8 * n1], zo = z0[64 + 8 * n1];
        y0[8 * n1] = v[n1].x * silu_f(ze);
        y0[64 + 8 * n1] = v[n1].y * silu_f(zo);
      }
    }
    // The next iteration's first shared-memory writes (EX: warp-private; ZR: last read
    // before the barrier above) cannot race with this iteration's GB reads, because GB is
    // next written only after the next iteration's first barrier.
  }
}

// ================================================================ generic planes ====
// Any H, W: direct DFTs with twiddle tables in shared memory.  Slow (O(N) per output)
// but exact in structure; used for plane sizes without a radix kernel and as an
// independent CUDA cross-check of the radix kernel in the tests.
constexpr int GEN_THREADS = 256;

__global__ void __launch_bounds__(GEN_THREADS)
gated_spectral_generic(float* __restrict__ xz, const cf* __restrict__ khat,
                       const float4* __restrict__ gates, int T, int C, int H, int W) {
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
      const float4 g = gp[o];
      const cf k = khc[o];
      cf A = mk(k.x * g.x, k.y * g.x);
      cf U = mk(g.y * ax, g.y * ay);
      if (U.x * U.x + U.y * U.y < g.w * g.w) U = mk(g.w, 0.f);
      cf hs = cmul(A, St[o]);
      hs.x += U.x; hs.y += U.y;
      St[o] = hs;
      Fb[o] = mk(g.z * hs.x, g.z * hs.y);
    }
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
      xp[o] = acc * silu_f(zp[o]);
    }
  }
}

size_t generic_smem_bytes(int H, int W) {
  const int Wf = W / 2 + 1;
  size_t fl = ((size_t)H * W + 1) & ~(size_t)1;
  return fl * 4 + (size_t)(W + H + 3 * H * Wf) * sizeof(cf);
}

int launch_gated_spectral(const cssm_gated_desc& d, const cf* khat, const float* gates,
                          float* xz, cudaStream_t st) {
  const SpectralPath path = spectral_path(d.H, d.W);
  const int grid = d.B * d.C;
  if (path == PATH_R64) {
    const size_t smem = R64_SMEM_CF * sizeof(cf);
    cudaError_t e = cudaFuncSetAttribute(gated_spectral_r64,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    gated_spectral_r64<<<grid, R64_THREADS, smem, st>>>(
        xz, khat, reinterpret_cast<const float4*>(gates), d.T, d.C);
  } else {
    const size_t smem = generic_smem_bytes(d.H, d.W);
    if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(gated_spectral_generic,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    gated_spectral_generic<<<grid, GEN_THREADS, smem, st>>>(
        xz, khat, reinterpret_cast<const float4*>(gates), d.T, d.C, d.H, d.W);
  }
  return check_launch();
}

}  // namespace cssm
