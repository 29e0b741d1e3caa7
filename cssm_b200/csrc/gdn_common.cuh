// Per-bin delta-rule update shared by the GDN spectral kernels.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

namespace cssm {

// One output row v of the d_v x d_k state at one frequency bin:
//   d = sum_j conj(k_j) S_j;  S_i <- aw*(S_i - beta*k_i*d) + beta*v*conj(k_i);  o = sum_i S_i q_i
// with aw = alpha * W_hat.  S points at S[v][0]; consecutive i are `ss` elements apart.
// READ = false skips the readout (returns 0); the state arithmetic is the same.
template <int DK, bool READ = true>
__device__ __forceinline__ cf gdn_bin_update_t(cf* S, size_t ss, const cf* kk, const cf* qq, cf vv,
                                               cf aw, float beta) {
  cf s[DK];
  cf d = mk(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < DK; ++j) {
    s[j] = S[j * ss];
    const cf p = cmulc(s[j], kk[j]);
    d.x += p.x; d.y += p.y;
  }
  cf o = mk(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const cf kd = cmul(kk[i], d);
    const cf inner = mk(s[i].x - beta * kd.x, s[i].y - beta * kd.y);
    cf n = cmul(aw, inner);
    const cf wr = cmulc(vv, kk[i]);
    n.x += beta * wr.x; n.y += beta * wr.y;
    S[i * ss] = n;
    if (READ) {
      const cf oq = cmul(n, qq[i]);
      o.x += oq.x; o.y += oq.y;
    }
  }
  return o;
}

// Same update on a state row that the caller has already loaded into registers (s) and will
// store itself: lets the caller batch the loads of several bins ahead of the stores.
template <int DK, bool READ = true>
__device__ __forceinline__ cf gdn_bin_update_regs(cf (&s)[DK], const cf* kk, const cf* qq, cf vv,
                                                  cf aw, float beta) {
  cf d = mk(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < DK; ++j) {
    const cf p = cmulc(s[j], kk[j]);
    d.x += p.x; d.y += p.y;
  }
  cf o = mk(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const cf kd = cmul(kk[i], d);
    const cf inner = mk(s[i].x - beta * kd.x, s[i].y - beta * kd.y);
    cf n = cmul(aw, inner);
    const cf wr = cmulc(vv, kk[i]);
    n.x += beta * wr.x; n.y += beta * wr.y;
    s[i] = n;
    if (READ) {
      const cf oq = cmul(n, qq[i]);
      o.x += oq.x; o.y += oq.y;
    }
  }
  return o;
}

__device__ __forceinline__ float bf16r(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// Static-image fast path (cssm.py:4353-4683): q, k, v of the bin are the same for all T steps,
// only the gates {alpha_t, beta_t} (ab[t * ab_stride]) vary.  Runs the whole scan of one state row
//   S_i <- bf16( sum_j bf16(M_t[i][j]) S_j + bf16(beta_t v conj(k_i)) ),
//   M_t[i][j] = alpha_t W_hat (delta_ij - beta_t k_i conj(k_j)),
// with M_t, Delta_t and the carry rounded to bfloat16 (real and imaginary parts) and the products
// accumulated in fp32, as the reference's linear-split scan does, and returns o = sum_i S_i q_i.
template <int DK>
__device__ __forceinline__ cf gdn_bin_static(const cf* kk, const cf* qq, cf vv, cf wh,
                                             const float2* __restrict__ ab, size_t ab_stride, int T) {
  cf K[DK][DK], vk[DK], s[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    vk[i] = cmulc(vv, kk[i]);
    s[i] = mk(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < DK; ++j) K[i][j] = cmulc(kk[i], kk[j]);
  }
  for (int t = 0; t < T; ++t) {
    const float2 g = __ldg(ab + (size_t)t * ab_stride);
    const cf aw = mk(g.x * wh.x, g.x * wh.y);
    cf n[DK];
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      float ar = bf16r(g.y * vk[i].x), ai = bf16r(g.y * vk[i].y);
#pragma unroll
      for (int j = 0; j < DK; ++j) {
        const cf inner = mk((i == j ? 1.f : 0.f) - g.y * K[i][j].x, -g.y * K[i][j].y);
        const cf m = cmul(aw, inner);
        const float mr = bf16r(m.x), mi = bf16r(m.y);
        ar += mr * s[j].x - mi * s[j].y;
        ai += mr * s[j].y + mi * s[j].x;
      }
      n[i] = mk(bf16r(ar), bf16r(ai));
    }
#pragma unroll
    for (int i = 0; i < DK; ++i) s[i] = n[i];
  }
  cf o = mk(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const cf oq = cmul(s[i], qq[i]);
    o.x += oq.x; o.y += oq.y;
  }
  return o;
}

}  // namespace cssm
