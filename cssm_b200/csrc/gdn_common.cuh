// Per-bin delta-rule update shared by the GDN spectral kernels.
#pragma once
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

__device__ __forceinline__ cf gdn_bin_update_r64(cf* S, size_t ss, const cf* kk, const cf* qq, cf vv,
                                                 cf aw, float beta) {
  return gdn_bin_update_t<4>(S, ss, kk, qq, vv, aw, beta);
}

}  // namespace cssm
