// Fused spectral kernels of the GDN block.  One CTA per (batch, head) walks t = 0..T-1:
// rfft2 of the head's q, k, v planes -> spectral / key L2 norms -> per-bin delta-rule update
//   d      = sum_j conj(k_j) S[v][j]
//   S[v][i] = alpha*W_hat*(S[v][i] - beta*k_i*d) + beta*v_v*conj(k_i)        (cssm.py:4911-4958)
//   o[v]   = sum_i S[v][i] q_i                                               (cssm.py:4998-5000)
// -> irfft2 of the d_v output planes, written over the v planes.
// M_t and Delta_t are never materialised.  The d_v x d_k complex state per bin does not fit one
// SM for 64x64 planes (270 KB), so it lives in a global scratch that stays L2-resident while
// its CTA runs (each CTA touches only its own 270 KB).
#include "fft.cuh"
#include "kernels.cuh"
#include "gdn_common.cuh"
#include "generic_dft.cuh"

namespace cssm {

constexpr int GDN_MAXDK = 4;

template <bool READ>
__device__ __forceinline__ cf gdn_bin_update(cf* S, size_t ss, int dk, const cf* kk, const cf* qq,
                                             cf vv, cf aw, float beta) {
  switch (dk) {
    case 1: return gdn_bin_update_t<1, READ>(S, ss, kk, qq, vv, aw, beta);
    case 2: return gdn_bin_update_t<2, READ>(S, ss, kk, qq, vv, aw, beta);
    case 3: return gdn_bin_update_t<3, READ>(S, ss, kk, qq, vv, aw, beta);
    default: return gdn_bin_update_t<4, READ>(S, ss, kk, qq, vv, aw, beta);
  }
}

// ================================================================ generic planes ====
__global__ void __launch_bounds__(GG_THREADS) gdn_spectral_generic(const GdnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.H, W = a.W, dk = a.dk;
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf;
  float* xs = reinterpret_cast<float*>(smem_raw);
  cf* twW = reinterpret_cast<cf*>(xs + ((HW + 1) & ~1));
  cf* twH = twW + W;
  cf* Rb = twH + H;
  cf* Fb = Rb + NB;
  cf* SK = Fb + NB;                 // [dk][NB] normalised keys
  cf* SQ = SK + (size_t)dk * NB;    // [dk][NB] normalised queries
  __shared__ float red[GG_THREADS / 32];

  const int tid = threadIdx.x;
  const int nh = a.C / dk;
  const int b = blockIdx.x / nh, hd = blockIdx.x % nh;
  for (int i = tid; i < W; i += GG_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)W, &s, &co); twW[i] = mk(co, s);
  }
  for (int i = tid; i < H; i += GG_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)H, &s, &co); twH[i] = mk(co, s);
  }
  cf* S = a.state + (size_t)blockIdx.x * dk * dk * NB;
  if (!a.static_image)
    for (int i = tid; i < dk * dk * NB; i += GG_THREADS) S[i] = mk(0.f, 0.f);
  const cf* wh = a.what + (size_t)hd * NB;
  const float invHW = 1.0f / (float)HW;
  const int Tdata = a.static_image ? 1 : a.T;      // frames of q, k, v per batch element

  for (int t = 0; t < Tdata; ++t) {
    const size_t frame = (size_t)(b * Tdata + t);
    float* base = a.qkv + frame * 3 * a.C * HW;
    const bool emit = !a.last_only || t == Tdata - 1;       // same for the whole CTA
    float nq[GDN_MAXDK], nk[GDN_MAXDK];
    for (int i = 0; i < dk; ++i) {
      float p = 0.f;
      nq[i] = 1.f;
      if (emit) {                                            // q is only needed for the readout
        gen_fwd_plane(base + (size_t)(hd * dk + i) * HW, xs, Rb, SQ + (size_t)i * NB, twW, twH, H, W);
        for (int o = tid; o < NB; o += GG_THREADS) { const cf z = SQ[(size_t)i * NB + o]; p += z.x * z.x + z.y * z.y; }
        nq[i] = a.use_l2 ? rsqrtf(block_sum(p, red) + 1e-6f) : 1.f;
      }
      gen_fwd_plane(base + (size_t)(a.C + hd * dk + i) * HW, xs, Rb, SK + (size_t)i * NB, twW, twH, H, W);
      p = 0.f;
      for (int o = tid; o < NB; o += GG_THREADS) { const cf z = SK[(size_t)i * NB + o]; p += z.x * z.x + z.y * z.y; }
      nk[i] = a.use_l2 ? rsqrtf(block_sum(p, red) + 1e-6f) : 1.f;
    }
    // normalise in place (each thread its own bins)
    for (int o = tid; o < NB; o += GG_THREADS) {
      float ks = 0.f;
      cf kv[GDN_MAXDK];
      for (int i = 0; i < dk; ++i) {
        const cf z = SK[(size_t)i * NB + o];
        kv[i] = mk(z.x * nk[i], z.y * nk[i]);
        ks += kv[i].x * kv[i].x + kv[i].y * kv[i].y;
        if (emit) {
          const cf q = SQ[(size_t)i * NB + o];
          SQ[(size_t)i * NB + o] = mk(q.x * nq[i], q.y * nq[i]);
        }
      }
      const float kn = rsqrtf(ks + 1e-6f);
      for (int i = 0; i < dk; ++i) SK[(size_t)i * NB + o] = mk(kv[i].x * kn, kv[i].y * kn);
    }
    const float2* ab = a.ab + ((a.static_image ? (size_t)b * a.T : frame) * a.ab_heads + (a.ab_heads > 1 ? hd : 0)) * NB;
    for (int v = 0; v < dk; ++v) {
      float* vplane = base + (size_t)(2 * a.C + hd * dk + v) * HW;
      gen_fwd_plane(vplane, xs, Rb, Fb, twW, twH, H, W);
      for (int o = tid; o < NB; o += GG_THREADS) {
        cf kk[GDN_MAXDK], qq[GDN_MAXDK];
        for (int i = 0; i < dk; ++i) { kk[i] = SK[(size_t)i * NB + o]; qq[i] = SQ[(size_t)i * NB + o]; }
        if (a.static_image) {
          cf ov;
          switch (dk) {
            case 1: ov = gdn_bin_static<1>(kk, qq, Fb[o], wh[o], ab + o, (size_t)a.ab_heads * NB, a.T); break;
            case 2: ov = gdn_bin_static<2>(kk, qq, Fb[o], wh[o], ab + o, (size_t)a.ab_heads * NB, a.T); break;
            case 3: ov = gdn_bin_static<3>(kk, qq, Fb[o], wh[o], ab + o, (size_t)a.ab_heads * NB, a.T); break;
            default: ov = gdn_bin_static<4>(kk, qq, Fb[o], wh[o], ab + o, (size_t)a.ab_heads * NB, a.T); break;
          }
          Fb[o] = mk(ov.x * invHW, ov.y * invHW);
          continue;
        }
        const float2 g = ab[o];
        const cf w = wh[o];
        const cf aw = mk(g.x * w.x, g.x * w.y);
        if (emit) {
          const cf ov = gdn_bin_update<true>(S + (size_t)v * dk * NB + o, NB, dk, kk, qq, Fb[o], aw, g.y);
          Fb[o] = mk(ov.x * invHW, ov.y * invHW);
        } else {
          gdn_bin_update<false>(S + (size_t)v * dk * NB + o, NB, dk, kk, qq, Fb[o], aw, g.y);
        }
      }
      if (!emit) continue;
      __syncthreads();
      for (int o = tid; o < NB; o += GG_THREADS) {
        const int h = o / Wf, kw = o % Wf;
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
      __syncthreads();
      const int kmax = (W - 1) / 2;
      for (int o = tid; o < HW; o += GG_THREADS) {
        const int h = o / W, w = o % W;
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
        vplane[o] = acc + 2.f * s2;
      }
    }
  }
}

size_t gdn_generic_smem_bytes(int H, int W, int dk) {
  const size_t Wf = W / 2 + 1, NB = (size_t)H * Wf;
  const size_t fl = ((size_t)H * W + 1) & ~(size_t)1;
  return fl * 4 + (W + H + 2 * NB + 2 * dk * NB) * sizeof(cf);
}

int launch_gdn_spectral_r64(const GdnSpectralArgs& a, cudaStream_t st);
int launch_gdn_spectral_r32(const GdnSpectralArgs& a, cudaStream_t st);

int launch_gdn_spectral(const GdnSpectralArgs& a, cudaStream_t st) {
  if (a.dk < 1 || a.dk > GDN_MAXDK || a.C % a.dk != 0) return CSSM_ERR_UNSUPPORTED;
  if (spectral_path(a.H, a.W) == PATH_R64 && a.dk == 4) return launch_gdn_spectral_r64(a, st);
  if (spectral_path(a.H, a.W) == PATH_R32 && a.dk == 4) return launch_gdn_spectral_r32(a, st);
  const size_t smem = gdn_generic_smem_bytes(a.H, a.W, a.dk);
  if (smem > 220 * 1024) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(gdn_spectral_generic,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  gdn_spectral_generic<<<a.B * (a.C / a.dk), GG_THREADS, smem, st>>>(a);
  return check_launch();
}

}  // namespace cssm
