// Fused spectral kernel of the DeltaNetCSSM block for 32x32 planes.  One CTA of 288 threads per
// (batch, group of four channels) walks t = 0..T-1; the four q planes, the four k planes and the
// four v planes of the group are each transformed side by side (r32.cuh geometry: plane = group / 17
// in the column passes).  Per step:
//   pass 0 (q), pass 1 (k times B_k): rows, columns -> the spectra wait in lane-private shared-memory
//     slots, sum |.|^2 per plane (the L2 norms over the half spectrum);
//   pass 2 (v times B_v): rows, columns -> per bin A = squash(alpha W_hat (1 - beta |k|^2)),
//     U = beta v conj(k), h = A h + U, o = C_gate h q -> inverse columns, inverse rows -> the output
//     planes over the v planes.
// The state h (8 bins per lane) stays in registers for the whole sequence.  The rows of the next pass's
// planes are fetched one pass ahead.
#include "r32.cuh"
#include "kernels.cuh"

namespace cssm {

constexpr int D32_THREADS = 288;
constexpr int D32_ZRS = 36, D32_GBS = 18;
constexpr int D32_EX_CF = 72 * EX32_STRIDE;
constexpr int D32_ZR_CF = 4 * 16 * D32_ZRS;
constexpr int D32_GB_CF = 4 * 32 * D32_GBS;
constexpr int D32_SPEC_CF = 2 * 8 * D32_THREADS;       // [q, k][r][thread]
constexpr int D32_SMEM_BYTES = (D32_EX_CF + D32_ZR_CF + D32_GB_CF + D32_SPEC_CF) * 8;

__global__ void __launch_bounds__(D32_THREADS, 2) deltanet_spectral_r32(const DnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZR = EX + D32_EX_CF;
  cf* GB = ZR + D32_ZR_CF;
  cf* SQ = GB + D32_GB_CF;                               // q spectrum, lane-private slots
  cf* SK = SQ + 8 * D32_THREADS;                         // gated k spectrum
  __shared__ float red[9][8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = lane & 3, g8 = lane >> 2;
  const int grp = warp * 8 + g8;
  cf* exg = EX + grp * EX32_STRIDE;
  const bool row_on = warp < 8;
  const bool col_warp = warp < 9, col_on = grp < 68;
  constexpr int HW = 1024, NB = 32 * 17;
  const int cgroups = a.C >> 2;
  const int b = blockIdx.x / cgroups, c0 = (blockIdx.x % cgroups) << 2;

  cf tw[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float s, co;
    sincospif(-(float)(q * k) / 16.0f, &s, &co);
    tw[k] = mk(co, s);
  }
  const int rpl = grp >> 4, rpair = grp & 15;
  const int roff = (2 * rpair) * 32 + q;
  const int cpl = col_on ? grp / 17 : 0, kw = col_on ? grp % 17 : 0;
  const int kneg = (32 - kw) & 31;
  const int par = q & 1, ph = q >> 1;
  const int boff = (kw << 2) + q;                        // the lane's first bin; register r adds r * 68
  const cf* whp = a.what + (size_t)(c0 + cpl) * NB + boff;
  const float floor_mag = a.goom_floor ? 1e-7f : 0.f;
  const bool chan = a.chan != nullptr;                   // same for the whole grid
  const float invHW = 1.0f / (float)HW;

  cf hst[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) hst[r] = mk(0.f, 0.f);

  auto rows_of = [&](int t, int pass) -> const float* {
    return a.qkv + ((size_t)(b * a.T + t) * 3 * a.C + (size_t)pass * a.C + c0 + rpl) * HW + roff;
  };
  cf nx[8];
  if (row_on) {
    const float* r0 = rows_of(0, 0);
#pragma unroll
    for (int m = 0; m < 8; ++m) nx[m] = mk(r0[4 * m], r0[32 + 4 * m]);
  }
  for (int t = 0; t < a.T; ++t) {
    const size_t frame = (size_t)(b * a.T + t);
    float* base = a.qkv + frame * 3 * a.C * HW;
    const size_t gbase = frame * NB + boff;
    float ssq[2] = {0.f, 0.f};
    cf v[8];
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      __syncthreads();                       // ZR free (previous column pass finished)
      if (row_on) {
        cf u[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) u[m] = nx[m];
        // the v planes of this step are overwritten by its output at the end of the step, after
        // this prefetch of the next step's q planes has long been consumed
        const int nt = pass < 2 ? t : t + 1;
        if (nt < a.T) {
          const float* r0 = rows_of(nt, pass < 2 ? pass + 1 : 0);
#pragma unroll
          for (int m = 0; m < 8; ++m) nx[m] = mk(r0[4 * m], r0[32 + 4 * m]);
        }
        fft32_fwd(u, tw, exg, q);
        cf* zr = ZR + (rpl * 16 + rpair) * D32_ZRS;
#pragma unroll
        for (int r = 0; r < 8; ++r) zr[q + 4 * (r >> 2) + 8 * (r & 3)] = u[r];
      }
      __syncthreads();
      if (col_warp) {
        const cf* zr = ZR + (cpl * 16) * D32_ZRS;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const cf z1 = zr[(ph + 2 * m) * D32_ZRS + kw];
          const cf z2 = zr[(ph + 2 * m) * D32_ZRS + kneg];
          v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
                     : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
        }
        fft32_fwd(v, tw, exg, q);
        if (pass < 2) {
          float acc = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            cf z = v[r];
            if (pass == 1) {
              const float bk = !col_on ? 0.f : (chan ? 1.f : __ldg(&a.abkv[gbase + r * 68].z));
              z = mk(z.x * bk, z.y * bk);
            }
            (pass == 0 ? SQ : SK)[r * D32_THREADS + tid] = z;
            if (col_on) acc += z.x * z.x + z.y * z.y;
          }
          if (pass == 0) ssq[0] = acc; else ssq[1] = acc;
        }
      }
    }
    // ---- per-plane sums over all bins: lanes of plane p live in groups 17p .. 17p+16 ----
#pragma unroll
    for (int pass = 0; pass < 2; ++pass)
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float c = (col_on && cpl == p) ? ssq[pass] : 0.f;
        for (int off = 16; off > 0; off >>= 1) c += __shfl_down_sync(0xffffffffu, c, off);
        if (lane == 0) red[warp][pass * 4 + p] = c;
      }
    __syncthreads();                          // red complete
    if (col_warp) {
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int w = 0; w < 9; ++w) { sq += red[w][cpl]; sk += red[w][4 + cpl]; }
      const float nq = rsqrtf(sq + 1e-6f), nk = rsqrtf(sk + 1e-6f);
      float2 ab = make_float2(0.f, 0.f);
      if (chan) ab = __ldg(&a.chan[frame * a.C + c0 + cpl]);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        float cgv = 0.f;
        cf w = mk(0.f, 0.f);
        if (col_on) {
          if (chan) {
            g = make_float4(ab.x, ab.y, 1.f, 1.f);
            cgv = invHW;
          } else {
            g = __ldg(&a.abkv[gbase + r * 68]);
            cgv = __ldg(&a.cg[gbase + r * 68]);
          }
          w = whp[r * 68];
        }
        const cf ks = SK[r * D32_THREADS + tid], qs = SQ[r * D32_THREADS + tid];
        const cf k = mk(ks.x * nk, ks.y * nk);
        const cf qq = mk(qs.x * nq, qs.y * nq);
        const cf vv = mk(v[r].x * g.w, v[r].y * g.w);
        const float kp = k.x * k.x + k.y * k.y;
        const float sc = g.x * (1.0f - g.y * kp);
        cf A = mk(w.x * sc, w.y * sc);
        const float am = sqrtf(A.x * A.x + A.y * A.y);
        const float sqv = a.rho / (1.0f + am);
        A = mk(A.x * sqv, A.y * sqv);
        if (am * sqv < floor_mag) A = mk(floor_mag, 0.f);
        cf U = cmulc(vv, k);
        U = mk(U.x * g.y, U.y * g.y);
        if (U.x * U.x + U.y * U.y < floor_mag * floor_mag) U = mk(floor_mag, 0.f);
        cf h = cmul(A, hst[r]);
        h.x += U.x; h.y += U.y;
        hst[r] = h;
        const cf oq = cmul(h, qq);
        v[r] = mk(oq.x * cgv, oq.y * cgv);
      }
      fft32_inv(v, tw, exg, q);
      cf* gb = GB + (cpl * 32) * D32_GBS;
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (col_on) gb[(q + 4 * m) * D32_GBS + kw] = v[m];
    }
    __syncthreads();
    // ---- inverse rows of the four output planes, written over the v planes ----
    if (row_on) {
      const cf* ge = GB + (rpl * 32 + 2 * rpair) * D32_GBS;
      const cf* go = ge + D32_GBS;
      cf u[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int k = q + 4 * (r >> 2) + 8 * (r & 3);
        const int kk = k <= 16 ? k : 32 - k;
        cf e = ge[kk], o = go[kk];
        if ((r == 0 || r == 2) && q == 0) { e.y = 0.f; o.y = 0.f; }
        u[r] = (k <= 16) ? mk(e.x - o.y, e.y + o.x) : mk(e.x + o.y, o.x - e.y);
      }
      fft32_inv(u, tw, exg, q);
      float* y0 = base + (size_t)(2 * a.C + c0 + rpl) * HW + roff;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        y0[4 * m] = u[m].x;
        y0[32 + 4 * m] = u[m].y;
      }
    }
  }
}

int launch_deltanet_spectral_r32(const DnSpectralArgs& a, cudaStream_t st) {
  if (a.H != 32 || a.W != 32 || a.C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(deltanet_spectral_r32,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, D32_SMEM_BYTES);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  deltanet_spectral_r32<<<a.B * (a.C / 4), D32_THREADS, D32_SMEM_BYTES, st>>>(a);
  return check_launch();
}

}  // namespace cssm
