// GDN fused spectral kernel for 32x32 planes, d_k = d_v = 4, with the whole matrix state on chip.
// One CTA (288 threads) per (batch, head).  The four planes of q, of k and of v are each
// transformed side by side (r32.cuh geometry: plane = group / 17 in column passes).  Per step:
//   1. q planes: rows, columns -> spectra parked in shared memory (SPEC), sum |.|^2 per plane
//   2. k planes: the same
//   3. v planes: rows, columns -> each column lane (v row = its plane) reads the 4 k and 4 q
//      values of its bins from SPEC, normalises them, updates its state row S[v][0..3] (shared
//      memory slots that only this lane ever touches: 8 bins x 4 complex per lane, 70 KB per
//      CTA), reads out o[v], inverse columns, inverse rows -> o planes over the v planes.
#include "r32.cuh"
#include "kernels.cuh"
#include "gdn_common.cuh"

namespace cssm {

constexpr int G32_THREADS = 288;
constexpr int G32_ZRS = 36, G32_GBS = 18;
constexpr int G32_EX_CF = 72 * EX32_STRIDE;
constexpr int G32_ZR_CF = 4 * 16 * G32_ZRS;
constexpr int G32_GB_CF = 4 * 32 * G32_GBS;
constexpr int G32_SPEC_CF = 8 * 8 * 17 * 4;            // [q planes 0-3, k planes 4-7][r][kw][q]
constexpr int G32_STATE_CF = 4 * 8 * G32_THREADS;      // [i][r][thread]
constexpr int G32_SMEM_BYTES = (G32_EX_CF + G32_ZR_CF + G32_GB_CF + G32_SPEC_CF + G32_STATE_CF) * 8;

// LAST: only the last step's output planes are produced (compile-time switch).
// STATIC: static-image fast path (one data frame per batch element, the T gate steps run per bin).
template <bool LAST, bool STATIC>
__global__ void __launch_bounds__(G32_THREADS, 1) gdn_spectral_r32(const GdnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZR = EX + G32_EX_CF;
  cf* GB = ZR + G32_ZR_CF;
  cf* SPEC = GB + G32_GB_CF;
  cf* ST = SPEC + G32_SPEC_CF;
  __shared__ float red[9][8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q = lane & 3, g8 = lane >> 2;
  const int grp = warp * 8 + g8;
  cf* exg = EX + grp * EX32_STRIDE;
  const bool row_on = warp < 8;
  const bool col_warp = warp < 9, col_on = grp < 68;
  constexpr int HW = 1024, NB = 32 * 17, DK = 4;
  const int nh = a.C / DK;
  const int b = blockIdx.x / nh, hd = blockIdx.x % nh;

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

  // state slots of this lane: ST[(i*8 + r)*288 + tid]
#pragma unroll
  for (int i = 0; i < 32; ++i) ST[i * G32_THREADS + tid] = mk(0.f, 0.f);
  cf wh[8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
    wh[r] = col_on ? a.what[(size_t)hd * NB + ((r * 17 + kw) << 2) + q] : mk(0.f, 0.f);
  const float invHW = 1.0f / (float)HW;

  const int Tdata = STATIC ? 1 : a.T;          // frames of q, k, v per batch element
  // rows of the NEXT pass's planes, fetched one pass ahead (the kernel runs nine warps per SM,
  // so a load issued where it is needed is not hidden by other warps)
  auto first_pass = [&](int t) -> int { return (LAST && t < Tdata - 1) ? 1 : 0; };
  auto rows_of = [&](int t, int pass) -> const float* {
    return a.qkv + ((size_t)(b * Tdata + t) * 3 * a.C + (size_t)pass * a.C + hd * DK + rpl) * HW + roff;
  };
  cf nx[8];
  if (row_on) {
    const float* r0 = rows_of(0, first_pass(0));
#pragma unroll
    for (int m = 0; m < 8; ++m) nx[m] = mk(r0[4 * m], r0[32 + 4 * m]);
  }
  for (int t = 0; t < Tdata; ++t) {
    const size_t frame = (size_t)(b * Tdata + t);
    float* base = a.qkv + frame * 3 * a.C * HW;
    float ssq[2] = {0.f, 0.f};
    const bool emit = !LAST || t == Tdata - 1;       // same for the whole CTA
    cf v[8];
    // ---- passes 0 (q), 1 (k), 2 (v): forward transform of four planes at once ----
#pragma unroll 1
    for (int pass = emit ? 0 : 1; pass < 3; ++pass) {     // q is only needed for the readout
      __syncthreads();                       // ZR free (previous column pass finished)
      if (row_on) {
        cf u[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) u[m] = nx[m];
        // the v planes of this step are overwritten by its output at the end of the step, after
        // this prefetch of the next step's first planes (q or k) has long been consumed
        const int nt = pass < 2 ? t : t + 1;
        if (nt < Tdata) {
          const float* r0 = rows_of(nt, pass < 2 ? pass + 1 : first_pass(nt));
#pragma unroll
          for (int m = 0; m < 8; ++m) nx[m] = mk(r0[4 * m], r0[32 + 4 * m]);
        }
        fft32_fwd(u, tw, exg, q);
        cf* zr = ZR + (rpl * 16 + rpair) * G32_ZRS;
#pragma unroll
        for (int r = 0; r < 8; ++r) zr[q + 4 * (r >> 2) + 8 * (r & 3)] = u[r];
      }
      __syncthreads();
      if (col_warp) {
        const cf* zr = ZR + (cpl * 16) * G32_ZRS;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const cf z1 = zr[(ph + 2 * m) * G32_ZRS + kw];
          const cf z2 = zr[(ph + 2 * m) * G32_ZRS + kneg];
          v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
                     : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
        }
        fft32_fwd(v, tw, exg, q);
        if (pass < 2) {
          float acc = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            if (col_on) {
              SPEC[(((pass * 4 + cpl) * 8 + r) * 17 + kw) * 4 + q] = v[r];
              acc += v[r].x * v[r].x + v[r].y * v[r].y;
            }
          }
          if (pass == 0) ssq[0] = acc; else ssq[1] = acc;
        }
      }
    }
    // ---- per-plane sums over all bins: lanes of plane p live in groups 17p .. 17p+16 ----
    {
      // each lane contributes to red[warp][pass*4 + plane] through a warp-level segmented sum
#pragma unroll
      for (int pass = 0; pass < 2; ++pass)
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          float c = (col_on && cpl == p) ? ssq[pass] : 0.f;
          for (int off = 16; off > 0; off >>= 1) c += __shfl_down_sync(0xffffffffu, c, off);
          if (lane == 0) red[warp][pass * 4 + p] = c;
        }
    }
    __syncthreads();                          // SPEC and red complete
    if (col_warp) {
      float nrm[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 9; ++w) s += red[w][p];
        nrm[p] = a.use_l2 ? rsqrtf(s + 1e-6f) : 1.f;
      }
      const float2* abp = a.ab + ((STATIC ? (size_t)b * a.T : frame) * a.ab_heads + (a.ab_heads > 1 ? hd : 0)) * NB + (kw << 2) + q;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        cf kk[4], qq[4];
        float ks = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const cf zq = SPEC[(((0 + i) * 8 + r) * 17 + kw) * 4 + q];
          const cf zk = SPEC[(((4 + i) * 8 + r) * 17 + kw) * 4 + q];
          qq[i] = mk(zq.x * nrm[i], zq.y * nrm[i]);
          kk[i] = mk(zk.x * nrm[4 + i], zk.y * nrm[4 + i]);
          ks += kk[i].x * kk[i].x + kk[i].y * kk[i].y;
        }
        const float kn = rsqrtf(ks + 1e-6f);
#pragma unroll
        for (int i = 0; i < 4; ++i) kk[i] = mk(kk[i].x * kn, kk[i].y * kn);
        cf o = mk(0.f, 0.f);
        if (STATIC) {
          if (col_on) o = gdn_bin_static<4>(kk, qq, v[r], wh[r], abp + r * (17 * 4), (size_t)a.ab_heads * NB, a.T);
        } else if (col_on) {
          const float2 g = abp[r * (17 * 4)];
          const cf aw = mk(g.x * wh[r].x, g.x * wh[r].y);
          if (emit)
            o = gdn_bin_update_t<4, true>(ST + r * G32_THREADS + tid, (size_t)8 * G32_THREADS, kk,
                                          qq, v[r], aw, g.y);
          else
            gdn_bin_update_t<4, false>(ST + r * G32_THREADS + tid, (size_t)8 * G32_THREADS, kk, qq,
                                       v[r], aw, g.y);
        }
        v[r] = mk(o.x * invHW, o.y * invHW);
      }
      if (emit) {
        fft32_inv(v, tw, exg, q);
        cf* gb = GB + (cpl * 32) * G32_GBS;
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (col_on) gb[(q + 4 * m) * G32_GBS + kw] = v[m];
      }
    }
    __syncthreads();
    // ---- inverse rows of the four output planes, written over the v planes ----
    if (row_on && emit) {
      const cf* ge = GB + (rpl * 32 + 2 * rpair) * G32_GBS;
      const cf* go = ge + G32_GBS;
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
      float* y0 = base + (size_t)(2 * a.C + hd * DK + rpl) * HW + roff;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        y0[4 * m] = u[m].x;
        y0[32 + 4 * m] = u[m].y;
      }
    }
  }
}

int launch_gdn_spectral_r32(const GdnSpectralArgs& a, cudaStream_t st) {
  auto kern = a.static_image ? gdn_spectral_r32<false, true>
                             : (a.last_only ? gdn_spectral_r32<true, false> : gdn_spectral_r32<false, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       G32_SMEM_BYTES);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  kern<<<a.B * (a.C / 4), G32_THREADS, G32_SMEM_BYTES, st>>>(a);
  return check_launch();
}

}  // namespace cssm
