// Building blocks of the 64x64 real 2-D FFT split over a 288-thread CTA (9 warps).
// lane = sub + 4*a; grp = 4*warp + sub is a row pair (row passes, warps 0..7) or a
// half-spectrum column kw (column passes, warps 0..8, valid when grp <= 32).
// After r64_col_fwd a lane holds bins kh = a + 8*q (q = 0..7) of column grp.
#pragma once
#include "fft.cuh"

namespace cssm {

constexpr int R64_NT = 288;
constexpr int R64_ZRS = 68;    // cf per packed row pair in ZR
constexpr int R64_GBS = 34;    // cf per spatial row in GB
constexpr int R64_EX_CF = 36 * EX_GROUP_STRIDE;
constexpr int R64_ZR_CF = 32 * R64_ZRS;
constexpr int R64_GB_CF = 64 * R64_GBS;

struct R64Ctx {
  cf* EX; cf* ZR; cf* GB;
  cf* exg;
  int warp, lane, sub, a, grp;
  bool row_on, col_warp, col_on;
  cf tw[8];
};

__device__ __forceinline__ void r64_init(R64Ctx& c, cf* EX, cf* ZR, cf* GB) {
  const int tid = threadIdx.x;
  c.EX = EX; c.ZR = ZR; c.GB = GB;
  c.warp = tid >> 5; c.lane = tid & 31; c.sub = c.lane & 3; c.a = c.lane >> 2;
  c.grp = c.warp * 4 + c.sub;
  c.row_on = c.warp < 8; c.col_warp = c.warp < 9; c.col_on = c.grp <= 32;
  c.exg = EX + c.grp * EX_GROUP_STRIDE;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float s, co;
    sincospif(-(float)(c.a * k) / 32.0f, &s, &co);
    c.tw[k] = mk(co, s);
  }
}

// rows: two real rows of `plane` as one complex FFT -> ZR.  Call from all threads; the
// caller places __syncthreads() after it.
__device__ __forceinline__ void r64_row_fwd(const R64Ctx& c, const float* __restrict__ plane) {
  if (c.row_on) {
    cf v[8];
    const float* r0 = plane + (2 * c.grp) * 64 + c.a;
#pragma unroll
    for (int m = 0; m < 8; ++m) v[m] = mk(r0[8 * m], r0[64 + 8 * m]);
    fft64_lane8<false>(v, c.tw, c.exg, c.a);
#pragma unroll
    for (int k2 = 0; k2 < 8; ++k2) c.ZR[c.grp * R64_ZRS + c.a + 8 * k2] = v[k2];
  }
}

// the same with the row values already in registers: v[m] = (x[2*grp][a+8m], x[2*grp+1][a+8m])
__device__ __forceinline__ void r64_row_fwd_regs(const R64Ctx& c, cf (&v)[8]) {
  if (c.row_on) {
    fft64_lane8<false>(v, c.tw, c.exg, c.a);
#pragma unroll
    for (int k2 = 0; k2 < 8; ++k2) c.ZR[c.grp * R64_ZRS + c.a + 8 * k2] = v[k2];
  }
}
__device__ __forceinline__ void r64_load_rows(const R64Ctx& c, const float* __restrict__ plane,
                                              cf (&v)[8]) {
  if (c.row_on) {
    const float* r0 = plane + (2 * c.grp) * 64 + c.a;
#pragma unroll
    for (int m = 0; m < 8; ++m) v[m] = mk(r0[8 * m], r0[64 + 8 * m]);
  }
}

// columns: Hermitian separation folded into the loads, then the column FFT.
// Only meaningful when c.col_warp; lanes with !col_on compute on in-bounds scratch.
__device__ __forceinline__ void r64_col_fwd(const R64Ctx& c, cf (&v)[8]) {
  const int par = c.a & 1, ph = c.a >> 1;
  const int kneg = (64 - c.grp) & 63;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const cf z1 = c.ZR[(ph + 4 * m) * R64_ZRS + c.grp];
    const cf z2 = c.ZR[(ph + 4 * m) * R64_ZRS + kneg];
    v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
               : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
  }
  fft64_lane8<false>(v, c.tw, c.exg, c.a);
}

// inverse columns of v (bins a + 8q) -> GB[h][kw].  The caller syncs afterwards.
__device__ __forceinline__ void r64_col_inv(const R64Ctx& c, cf (&v)[8]) {
  fft64_lane8<true>(v, c.tw, c.exg, c.a);
#pragma unroll
  for (int n1 = 0; n1 < 8; ++n1)
    if (c.col_on) c.GB[(c.a + 8 * n1) * R64_GBS + c.grp] = v[n1];
}

// inverse rows (C2R; imaginary parts of the DC and Nyquist columns are ignored, as irfft2
// does): on return v[n1] = (y[2*grp][a + 8*n1], y[2*grp + 1][a + 8*n1]).  Row warps only.
__device__ __forceinline__ void r64_row_inv(const R64Ctx& c, cf (&v)[8]) {
  const cf* ge = c.GB + (2 * c.grp) * R64_GBS;
  const cf* go = ge + R64_GBS;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int n = c.a + 8 * m;
    const int k = n <= 32 ? n : 64 - n;
    cf e = ge[k], o = go[k];
    if ((m == 0 || m == 4) && c.a == 0) { e.y = 0.f; o.y = 0.f; }
    v[m] = (n <= 32) ? mk(e.x - o.y, e.y + o.x) : mk(e.x + o.y, o.x - e.y);
  }
  fft64_lane8<true>(v, c.tw, c.exg, c.a);
}

}  // namespace cssm
