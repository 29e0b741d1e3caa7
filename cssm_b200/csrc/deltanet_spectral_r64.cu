// Fused spectral kernel of the DeltaNetCSSM block for 64x64 planes.  One CTA of 288 threads per
// (batch, channel) walks t = 0..T-1:
//   rfft2 of the q, k, v planes (radix-8 x radix-8 split over 8 lanes, rows then columns)
//   -> k times B_k; L2 norms of q and k over the half-spectrum; v times B_v
//   -> per bin: A = squash(alpha W_hat (1 - beta |k|^2)), U = beta v conj(k), h = A h + U
//   -> C_gate h q -> irfft2, written over the v plane.
// The state h (8 bins per lane) stays in registers for the whole sequence; the q and k spectra
// wait in shared memory while the next plane is transformed.  The rows of the next plane are
// fetched into registers while the current one is transformed.
#include <cuda_runtime.h>
#include "r64.cuh"
#include "kernels.cuh"

namespace cssm {

constexpr int DN64_SMEM_BYTES = (R64_EX_CF + R64_ZR_CF + R64_GB_CF + 2 * 8 * R64_NT) * (int)sizeof(cf);

__global__ void __launch_bounds__(R64_NT, 2) deltanet_spectral_r64(const DnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* SQ = EX + R64_EX_CF + R64_ZR_CF + R64_GB_CF;      // [8][288] q spectrum, lane-private slots
  cf* SK = SQ + 8 * R64_NT;                             // [8][288] gated k spectrum
  __shared__ float red[2 * 9];
  R64Ctx c;
  r64_init(c, EX, EX + R64_EX_CF, EX + R64_EX_CF + R64_ZR_CF);

  const int tid = threadIdx.x;
  const int b = blockIdx.x / a.C, ch = blockIdx.x % a.C;
  constexpr int HW = 64 * 64, NB = 64 * 33;
  const size_t fstride = (size_t)3 * a.C * HW;
  float* q0 = a.qkv + (size_t)(b * a.T) * fstride + (size_t)ch * HW;       // q plane of step 0
  const size_t koff = (size_t)a.C * HW, voff = 2 * koff;
  const int boff = (c.grp << 3) + c.a;                   // the lane's first bin (kh = a, kw = grp)
  const cf* whp = a.what + (size_t)ch * NB + boff;
  const float floor_mag = a.goom_floor ? 1e-7f : 0.f;
  const bool chan = a.chan != nullptr;                   // same for the whole grid
  const int roff = (2 * c.grp) * 64 + c.a;

  cf hst[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) hst[q] = mk(0.f, 0.f);
  cf rows[8];
  r64_load_rows(c, q0, rows);

  for (int t = 0; t < a.T; ++t) {
    float* qp = q0 + (size_t)t * fstride;
    const size_t gbase = (size_t)(b * a.T + t) * NB + boff;
    float pq = 0.f, pk = 0.f;

    // ---- q ----
    r64_row_fwd_regs(c, rows);
    r64_load_rows(c, qp + koff, rows);
    __syncthreads();
    if (c.col_warp) {
      cf v[8];
      r64_col_fwd(c, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        SQ[q * R64_NT + tid] = v[q];
        if (c.col_on) pq += v[q].x * v[q].x + v[q].y * v[q].y;
      }
    }
    __syncthreads();

    // ---- k ----
    r64_row_fwd_regs(c, rows);
    r64_load_rows(c, qp + voff, rows);
    __syncthreads();
    if (c.col_warp) {
      cf v[8];
      r64_col_fwd(c, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float bk = !c.col_on ? 0.f : (chan ? 1.f : __ldg(&a.abkv[gbase + q * (33 * 8)].z));
        v[q] = mk(v[q].x * bk, v[q].y * bk);
        SK[q * R64_NT + tid] = v[q];
        pk += v[q].x * v[q].x + v[q].y * v[q].y;
      }
      for (int off = 16; off > 0; off >>= 1) {
        pq += __shfl_down_sync(0xffffffffu, pq, off);
        pk += __shfl_down_sync(0xffffffffu, pk, off);
      }
      if (c.lane == 0) { red[2 * c.warp] = pq; red[2 * c.warp + 1] = pk; }
    }
    __syncthreads();

    // ---- v, delta rule, inverse columns ----
    r64_row_fwd_regs(c, rows);
    if (t + 1 < a.T) r64_load_rows(c, qp + fstride, rows);
    __syncthreads();
    if (c.col_warp) {
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int w = 0; w < 9; ++w) { sq += red[2 * w]; sk += red[2 * w + 1]; }
      const float nq = rsqrtf(sq + 1e-6f), nk = rsqrtf(sk + 1e-6f);
      cf v[8];
      r64_col_fwd(c, v);
      float2 ab = make_float2(0.f, 0.f);
      if (chan) ab = __ldg(&a.chan[(size_t)(b * a.T + t) * a.C + ch]);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        float cgv = 0.f;
        cf w = mk(0.f, 0.f);
        if (c.col_on) {
          if (chan) {
            g = make_float4(ab.x, ab.y, 1.f, 1.f);
            cgv = 1.0f / (float)HW;
          } else {
            g = __ldg(&a.abkv[gbase + q * (33 * 8)]);
            cgv = __ldg(&a.cg[gbase + q * (33 * 8)]);
          }
          w = whp[q * (33 * 8)];
        }
        const cf ks = SK[q * R64_NT + tid], qs = SQ[q * R64_NT + tid];
        const cf k = mk(ks.x * nk, ks.y * nk);
        const cf qq = mk(qs.x * nq, qs.y * nq);
        const cf vv = mk(v[q].x * g.w, v[q].y * g.w);
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
        cf h = cmul(A, hst[q]);
        h.x += U.x; h.y += U.y;
        hst[q] = h;
        const cf oq = cmul(h, qq);
        v[q] = mk(oq.x * cgv, oq.y * cgv);
      }
      r64_col_inv(c, v);
    }
    __syncthreads();

    // ---- inverse rows, store over the v plane ----
    if (c.row_on) {
      cf v[8];
      r64_row_inv(c, v);
      float* y0 = qp + voff + roff;
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1) {
        y0[8 * n1] = v[n1].x;
        y0[64 + 8 * n1] = v[n1].y;
      }
    }
    // the next iteration writes ZR (last read before the barrier above) and EX (warp-private);
    // GB is rewritten three barriers from here; red is rewritten two barriers from here
  }
}

int launch_deltanet_spectral_r64(const DnSpectralArgs& a, cudaStream_t st) {
  if (a.H != 64 || a.W != 64) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(deltanet_spectral_r64,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, DN64_SMEM_BYTES);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  deltanet_spectral_r64<<<a.B * a.C, R64_NT, DN64_SMEM_BYTES, st>>>(a);
  return check_launch();
}

}  // namespace cssm
