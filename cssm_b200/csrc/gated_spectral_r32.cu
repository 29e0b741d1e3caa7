// Fused gated spectral kernel for 32x32 planes.  One CTA (288 threads) per (batch, group of four
// channels): same phase structure as the 64x64 kernel, with every 32-point FFT split over four
// lanes (r32.cuh) and four planes side by side so that the warps are full.
//   row passes   : 4 planes x 16 row pairs = 64 FFTs  -> warps 0..7
//   column passes: 4 planes x 17 columns   = 68 FFTs  -> warps 0..8 (groups 68..71 idle)
// A lane keeps the state of its 8 bins (kh = q + 4*(r>>2) + 8*(r&3)) in registers for all T.
#include "r32.cuh"
#include "kernels.cuh"

namespace cssm {

constexpr int R32_THREADS = 288;
constexpr int R32_ZRS = 36;     // cf per packed row pair
constexpr int R32_GBS = 18;     // cf per spatial row
constexpr int R32_EX_CF = 72 * EX32_STRIDE;
constexpr int R32_ZR_CF = 4 * 16 * R32_ZRS;
constexpr int R32_GB_CF = 4 * 32 * R32_GBS;
constexpr int R32_SMEM_BYTES = (R32_EX_CF + R32_ZR_CF + R32_GB_CF) * 8;

// LAST: only the last step's output planes are produced (compile-time switch).
// MODE 0: gate maps and z planes; 1: ungated recurrence S_t = K_hat S_{t-1} + X_hat_t (neither);
// 2: gate maps, no z planes; 3: as 2 with a per-(frame, channel) decay dchan[frame, c] on top of the maps.
template <bool LAST, int MODE>
__global__ void __launch_bounds__(R32_THREADS, 2)
gated_spectral_r32(float* __restrict__ xz, const cf* __restrict__ khat,
                   const float4* __restrict__ gates, int T, int C, const float* __restrict__ dchan) {
  constexpr int last_only = LAST ? 1 : 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZR = EX + R32_EX_CF;
  cf* GB = ZR + R32_ZR_CF;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = lane & 3, g8 = lane >> 2;
  const int grp = warp * 8 + g8;
  cf* exg = EX + grp * EX32_STRIDE;
  const bool row_on = warp < 8;
  const bool col_warp = warp < 9, col_on = grp < 68;
  const int cgroups = C >> 2;
  const int b = blockIdx.x / cgroups, c0 = (blockIdx.x % cgroups) << 2;
  constexpr int HW = 1024, NB = 32 * 17;

  cf tw[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float s, co;
    sincospif(-(float)(q * k) / 16.0f, &s, &co);
    tw[k] = mk(co, s);
  }
  // row role
  const int rpl = grp >> 4, rpair = grp & 15;
  const int roff = (2 * rpair) * 32 + q;
  // column role (clamped for the idle groups so that their shared-memory reads stay in bounds)
  const int cpl = col_on ? grp / 17 : 0, kw = col_on ? grp % 17 : 0;
  const int kneg = (32 - kw) & 31;
  const cf* khp = khat + (size_t)(c0 + cpl) * NB + (kw << 2) + q;

  cf hst[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) hst[r] = mk(0.f, 0.f);

  for (int t = 0; t < T; ++t) {
    const size_t frame = (size_t)(b * T + t);
    float* xp = xz + (frame * 2 * C + c0 + rpl) * HW;           // row role's plane
    const float* zp = xp + (size_t)C * HW;
    const bool emit = !last_only || t == T - 1;                  // same for the whole CTA

    // ---- forward rows ----
    if (row_on) {
      cf v[8];
      const float* r0 = xp + roff;
#pragma unroll
      for (int m = 0; m < 8; ++m) v[m] = mk(r0[4 * m], r0[32 + 4 * m]);   // plain loads: y overwrites this plane
      fft32_fwd(v, tw, exg, q);
      cf* zr = ZR + (rpl * 16 + rpair) * R32_ZRS;
#pragma unroll
      for (int r = 0; r < 8; ++r) zr[q + 4 * (r >> 2) + 8 * (r & 3)] = v[r];
    }
    __syncthreads();

    // ---- forward columns, recurrence, inverse columns ----
    if (col_warp) {
      float4 g[8];
      cf kh[8];
      const float4* gp = gates + frame * NB + (kw << 2) + q;
      const float dc = MODE == 3 ? __ldg(dchan + frame * C + c0 + cpl) : 1.f;   // per-(frame, channel) decay
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (MODE != 1) g[r] = col_on ? __ldg(gp + r * (17 * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE == 3) g[r].x *= dc;
        kh[r] = col_on ? khp[r * (17 * 4)] : mk(0.f, 0.f);
      }
      cf v[8];
      const int par = q & 1, ph = q >> 1;
      const cf* zr = ZR + (cpl * 16) * R32_ZRS;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const cf z1 = zr[(ph + 2 * m) * R32_ZRS + kw];
        const cf z2 = zr[(ph + 2 * m) * R32_ZRS + kneg];
        v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
                   : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
      }
      fft32_fwd(v, tw, exg, q);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (MODE == 1) {
          cf h = cmul(kh[r], hst[r]);
          h.x += v[r].x; h.y += v[r].y;
          hst[r] = h;
          v[r] = mk(h.x * (1.0f / HW), h.y * (1.0f / HW));
        } else {
          const cf A = mk(kh[r].x * g[r].x, kh[r].y * g[r].x);
          cf U = mk(g[r].y * v[r].x, g[r].y * v[r].y);
          if (U.x * U.x + U.y * U.y < g[r].w * g[r].w) U = mk(g[r].w, 0.f);
          cf h = cmul(A, hst[r]);
          h.x += U.x; h.y += U.y;
          hst[r] = h;
          v[r] = mk(g[r].z * h.x, g[r].z * h.y);
        }
      }
      if (emit) {
        fft32_inv(v, tw, exg, q);
        cf* gb = GB + (cpl * 32) * R32_GBS;
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (col_on) gb[(q + 4 * m) * R32_GBS + kw] = v[m];
      }
    }
    __syncthreads();

    // ---- inverse rows (C2R; imaginary parts of the DC and Nyquist columns ignored) ----
    if (row_on && emit) {
      float ze[8], zo[8];
      const float* z0 = zp + roff;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        ze[m] = MODE != 0 ? 1.f : __ldg(z0 + 4 * m);
        zo[m] = MODE != 0 ? 1.f : __ldg(z0 + 32 + 4 * m);
      }
      const cf* ge = GB + (rpl * 32 + 2 * rpair) * R32_GBS;
      const cf* go = ge + R32_GBS;
      cf v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int k = q + 4 * (r >> 2) + 8 * (r & 3);
        const int kk = k <= 16 ? k : 32 - k;
        cf e = ge[kk], o = go[kk];
        if ((r == 0 || r == 2) && q == 0) { e.y = 0.f; o.y = 0.f; }      // k = 0 and k = 16
        v[r] = (k <= 16) ? mk(e.x - o.y, e.y + o.x) : mk(e.x + o.y, o.x - e.y);
      }
      fft32_inv(v, tw, exg, q);
      float* y0 = xp + roff;
#pragma unroll
      for (int m = 0; m < 8; ++m) v[m] = mk(v[m].x * ze[m], v[m].y * zo[m]);
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        y0[4 * m] = v[m].x;
        y0[32 + 4 * m] = v[m].y;
      }
    }
    // the next iteration's first writes go to EX (warp-private) and ZR (last read before the
    // second barrier above); GB is next written after the next first barrier
  }
}

int launch_gated_spectral_r32(float* xz, const cf* khat, const float* gates, int B, int T, int C,
                              int last_only, int nogate, cudaStream_t st, const float* dchan) {
  auto kern = last_only ? gated_spectral_r32<true, 0> : gated_spectral_r32<false, 0>;
  if (nogate == 1) kern = last_only ? gated_spectral_r32<true, 1> : gated_spectral_r32<false, 1>;
  if (nogate == 2) kern = last_only ? gated_spectral_r32<true, 2> : gated_spectral_r32<false, 2>;
  if (nogate == 3) kern = last_only ? gated_spectral_r32<true, 3> : gated_spectral_r32<false, 3>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       R32_SMEM_BYTES);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  kern<<<B * (C / 4), R32_THREADS, R32_SMEM_BYTES, st>>>(
      xz, khat, reinterpret_cast<const float4*>(gates), T, C, dchan);
  return check_launch();
}

}  // namespace cssm
