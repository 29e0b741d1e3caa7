// GDN fused spectral kernel for 64x64 planes, d_k = d_v = 4.  One CTA (288 threads) per
// (batch, head).  Per step: the 8 q/k planes are transformed and their spectra parked in
// shared memory in the column lanes' own bin order; the norms are applied in place; then each
// of the 4 v planes is transformed, its state row updated and read out, and the output plane
// inverse-transformed over the v plane.
#include "r64.cuh"
#include "kernels.cuh"
#include "gdn_common.cuh"

namespace cssm {

constexpr int G64_SPEC_CF = 8 * 8 * R64_NT;     // [plane 0..7][q 0..7][thread]
constexpr int G64_SMEM_CF = R64_EX_CF + R64_ZR_CF + R64_GB_CF + G64_SPEC_CF;

// LAST: only the last step's output planes are produced (compile-time switch).
// STATIC: static-image fast path (one data frame per batch element, the T gate steps run per bin).
template <bool LAST, bool STATIC>
__global__ void __launch_bounds__(R64_NT, 1) gdn_spectral_r64(const GdnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZR = EX + R64_EX_CF;
  cf* GB = ZR + R64_ZR_CF;
  cf* SPEC = GB + R64_GB_CF;
  __shared__ float red[9][8];

  R64Ctx c;
  r64_init(c, EX, ZR, GB);
  const int tid = threadIdx.x;
  constexpr int HW = 4096, NB = 64 * 33, DK = 4;
  const int nh = a.C / DK;
  const int b = blockIdx.x / nh, hd = blockIdx.x % nh;
  const int Tdata = STATIC ? 1 : a.T;          // frames of q, k, v per batch element

  // state scratch: S[v][i][q][thread]; zero it (a thread only ever touches its own slots)
  cf* S = a.state + (size_t)blockIdx.x * DK * DK * NB;   // 16 * 2112 = 16 * 8 * 264 slots
  // lanes of column passes: slot index inside a (v,i) block is q*264 + (grp*8 + a), grp <= 32
  const int cslot = c.grp * 8 + c.a;
  if (c.col_on && !STATIC)
    for (int vi = 0; vi < DK * DK; ++vi)
#pragma unroll
      for (int q = 0; q < 8; ++q) S[(size_t)vi * NB + q * 264 + cslot] = mk(0.f, 0.f);

  cf wh[8];
#pragma unroll
  for (int q = 0; q < 8; ++q)
    wh[q] = c.col_on ? a.what[(size_t)hd * NB + ((q * 33 + c.grp) << 3) + c.a] : mk(0.f, 0.f);
  const float invHW = 1.0f / (float)HW;

  // plane idx 0..3 = q, 4..7 = k, 8..11 = v of step t; idx 12 = first plane of step t + 1
  // last_only: steps before the last one skip the q planes (their sequence starts at idx 4)
  auto first_of = [&](int t) -> int { return (LAST && t < Tdata - 1) ? 4 : 0; };
  auto plane_of = [&](int t, int idx) -> float* {
    if (idx >= 12) { ++t; idx = first_of(t); }
    if (t >= Tdata) { t = Tdata - 1; idx = 0; }             // harmless re-read past the end
    const size_t frame = (size_t)(b * Tdata + t);
    return a.qkv + (frame * 3 * a.C + (size_t)(idx >> 2) * a.C + hd * DK + (idx & 3)) * HW;
  };
  cf nx[8];                                   // rows of the NEXT plane, fetched one pass ahead
  r64_load_rows(c, plane_of(0, first_of(0)), nx);

  for (int t = 0; t < Tdata; ++t) {
    const size_t frame = (size_t)(b * Tdata + t);
    float* base = a.qkv + frame * 3 * a.C * HW;
    const bool emit = !LAST || t == Tdata - 1;       // same for the whole CTA
    float ssq[8];
#pragma unroll
    for (int p = 0; p < 4; ++p) ssq[p] = 0.f;
    // ---- q planes (p = 0..3) and k planes (p = 4..7) ----
#pragma unroll 1
    for (int p = first_of(t); p < 8; ++p) {
      __syncthreads();                       // ZR free (previous column pass finished)
      {
        cf cur[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) cur[m] = nx[m];
        r64_load_rows(c, plane_of(t, p + 1), nx);
        r64_row_fwd_regs(c, cur);
      }
      __syncthreads();
      float acc = 0.f;
      if (c.col_warp) {
        cf v[8];
        r64_col_fwd(c, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          SPEC[(p * 8 + q) * R64_NT + tid] = v[q];
          if (c.col_on) acc += v[q].x * v[q].x + v[q].y * v[q].y;
        }
      }
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
      // valid in lane 0 of each warp (ssq is indexed statically to stay in registers)
#pragma unroll
      for (int pp = 0; pp < 8; ++pp) if (pp == p) ssq[pp] = acc;
    }
    if (c.lane == 0)
#pragma unroll
      for (int p = 0; p < 8; ++p) red[c.warp][p] = ssq[p];
    __syncthreads();
    float nrm[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 9; ++w) s += red[w][p];
      nrm[p] = a.use_l2 ? rsqrtf(s + 1e-6f) : 1.f;
    }
    // ---- normalise own bins in place: q_hat = q*nq; k_hat = (k*nk) / sqrt(sum_i |.|^2 + 1e-6)
    if (c.col_warp) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        cf kv[4];
        float ks = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          cf z = SPEC[((4 + i) * 8 + q) * R64_NT + tid];
          kv[i] = mk(z.x * nrm[4 + i], z.y * nrm[4 + i]);
          ks += kv[i].x * kv[i].x + kv[i].y * kv[i].y;
          if (emit) {
            cf qq = SPEC[(i * 8 + q) * R64_NT + tid];
            SPEC[(i * 8 + q) * R64_NT + tid] = mk(qq.x * nrm[i], qq.y * nrm[i]);
          }
        }
        const float kn = rsqrtf(ks + 1e-6f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          SPEC[((4 + i) * 8 + q) * R64_NT + tid] = mk(kv[i].x * kn, kv[i].y * kn);
      }
    }
    // gates: of this frame, or (static path) of step 0 of this batch element's T steps
    const float2* abp = a.ab + ((STATIC ? (size_t)b * a.T : frame) * a.ab_heads + (a.ab_heads > 1 ? hd : 0)) * NB + (c.grp << 3) + c.a;
    // ---- v rows: transform, state update, readout, inverse transform over the v plane ----
#pragma unroll 1
    for (int vr = 0; vr < DK; ++vr) {
      float* vplane = base + (size_t)(2 * a.C + hd * DK + vr) * HW;
      __syncthreads();                       // ZR free; GB reads of the previous row finished
      {
        cf cur[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) cur[m] = nx[m];
        r64_load_rows(c, plane_of(t, 8 + vr + 1), nx);
        r64_row_fwd_regs(c, cur);
      }
      __syncthreads();
      if (c.col_warp) {
        // the state row of all 8 bins is fetched before the transform (the scratch is only
        // L2-resident) and written back after the last bin, so the loads are not pinned behind
        // the stores of the previous bin
        cf sreg[8][4];
        float2 gab[8];
        cf* srow = S + (size_t)(vr * DK) * NB + cslot;
        if (!STATIC) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              sreg[q][i] = c.col_on ? srow[(size_t)i * NB + q * 264] : mk(0.f, 0.f);
            gab[q] = c.col_on ? __ldg(abp + q * (33 * 8)) : make_float2(0.f, 0.f);
          }
        }
        cf v[8];
        r64_col_fwd(c, v);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          cf kk[4], qq[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            qq[i] = SPEC[(i * 8 + q) * R64_NT + tid];
            kk[i] = SPEC[((4 + i) * 8 + q) * R64_NT + tid];
          }
          if (STATIC) {
            cf o = mk(0.f, 0.f);
            if (c.col_on) o = gdn_bin_static<4>(kk, qq, v[q], wh[q], abp + q * (33 * 8), (size_t)a.ab_heads * NB, a.T);
            v[q] = mk(o.x * invHW, o.y * invHW);
            continue;
          }
          const cf aw = mk(gab[q].x * wh[q].x, gab[q].x * wh[q].y);
          if (emit) {
            const cf o = gdn_bin_update_regs<4, true>(sreg[q], kk, qq, v[q], aw, gab[q].y);
            v[q] = mk(o.x * invHW, o.y * invHW);
          } else {
            gdn_bin_update_regs<4, false>(sreg[q], kk, qq, v[q], aw, gab[q].y);
          }
        }
        if (c.col_on && !STATIC) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) srow[(size_t)i * NB + q * 264] = sreg[q][i];
        }
        if (emit) r64_col_inv(c, v);
      }
      __syncthreads();
      if (c.row_on && emit) {
        cf v[8];
        r64_row_inv(c, v);
        float* y0 = vplane + (2 * c.grp) * 64 + c.a;
#pragma unroll
        for (int n1 = 0; n1 < 8; ++n1) {
          y0[8 * n1] = v[n1].x;
          y0[64 + 8 * n1] = v[n1].y;
        }
      }
    }
  }
}

int launch_gdn_spectral_r64(const GdnSpectralArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)G64_SMEM_CF * sizeof(cf);
  auto kern = a.static_image ? gdn_spectral_r64<false, true>
                             : (a.last_only ? gdn_spectral_r64<true, false> : gdn_spectral_r64<false, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  kern<<<a.B * (a.C / 4), R64_NT, smem, st>>>(a);
  return check_launch();
}

}  // namespace cssm
