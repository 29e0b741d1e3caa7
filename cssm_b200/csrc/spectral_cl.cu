// Fused spectral kernel of the gated block for the small planes of the CSSM-SHViT stages
// (14 x 14 and 7 x 7) at T = 1, on bf16 channels-last activations:
//   y[n, p, c] = irfft2( C * floor((Delta + 1e-8) * B * rfft2(x[n, :, c])) )[p] * z[n, p, c]
// (at T = 1 the state is h_1 = U_1, so the kernel spectrum K_hat does not enter; z arrives already
// through SiLU).  TWO threads per (sample, channel) plane, 64 channels of one sample per CTA: in the
// row passes a thread owns half of the rows, in the column pass half of the spectrum columns.  The
// DFT twiddles are compile-time constants shared by every thread, so the transforms are straight
// FMA chains without shuffles; the 14-point complex DFTs of the column passes are split into two
// 7-point DFTs.  The half spectrum of the plane (N x (N/2+1) complex) waits in shared memory between
// the passes as fp16 pairs [bin][plane] (conflict-free; the row pass scales by 1/N so that the
// values stay in range, fp16's 11 significant bits are finer than the bf16 output): 55 KB per CTA
// instead of 84 KB with fp32, four CTAs = 16 warps per SM instead of 4 warps.  The input tile, the z
// tile and the output tile share one [pixel][64] bf16 buffer that is filled and drained with
// 16-byte accesses, so HBM sees x, z and y once each as full 128-byte rows.
#include <cuda_fp16.h>
#include "kernels.cuh"
#include "bf16_ops.cuh"

namespace cssm {

constexpr int SCL_PL = 64;             // planes (channels of one sample) per CTA
constexpr int SCL_TPB = 2 * SCL_PL;    // two threads per plane

template <int N> struct Tw;
template <> struct Tw<7> {
  static __device__ __forceinline__ float c(int i) {
    constexpr float t[7] = {1.000000000e+00f, 6.234898019e-01f, -2.225209340e-01f, -9.009688679e-01f,
                            -9.009688679e-01f, -2.225209340e-01f, 6.234898019e-01f};
    return t[i];
  }
  static __device__ __forceinline__ float s(int i) {
    constexpr float t[7] = {0.000000000e+00f, 7.818314825e-01f, 9.749279122e-01f, 4.338837391e-01f,
                            -4.338837391e-01f, -9.749279122e-01f, -7.818314825e-01f};
    return t[i];
  }
};
template <> struct Tw<14> {
  static __device__ __forceinline__ float c(int i) {
    constexpr float t[14] = {1.000000000e+00f, 9.009688679e-01f, 6.234898019e-01f, 2.225209340e-01f,
                             -2.225209340e-01f, -6.234898019e-01f, -9.009688679e-01f, -1.000000000e+00f,
                             -9.009688679e-01f, -6.234898019e-01f, -2.225209340e-01f, 2.225209340e-01f,
                             6.234898019e-01f, 9.009688679e-01f};
    return t[i];
  }
  static __device__ __forceinline__ float s(int i) {
    constexpr float t[14] = {0.000000000e+00f, 4.338837391e-01f, 7.818314825e-01f, 9.749279122e-01f,
                             9.749279122e-01f, 7.818314825e-01f, 4.338837391e-01f, 0.000000000e+00f,
                             -4.338837391e-01f, -7.818314825e-01f, -9.749279122e-01f, -9.749279122e-01f,
                             -7.818314825e-01f, -4.338837391e-01f};
    return t[i];
  }
};

// 7-point complex DFT, y[k] = sum_n x[n] e^{SIGN 2 pi i n k / 7}
template <int SIGN>
__device__ __forceinline__ void dft7c(const float (&xr)[7], const float (&xi)[7], float (&yr)[7],
                                      float (&yi)[7]) {
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    float ar = xr[0], ai = xi[0];
#pragma unroll
    for (int n = 1; n < 7; ++n) {
      const float c = Tw<7>::c((n * k) % 7), s = SIGN * Tw<7>::s((n * k) % 7);
      ar = fmaf(xr[n], c, ar); ar = fmaf(-xi[n], s, ar);
      ai = fmaf(xr[n], s, ai); ai = fmaf(xi[n], c, ai);
    }
    yr[k] = ar; yi[k] = ai;
  }
}

// N-point complex DFT in place (N = 7 direct; N = 14 as two 7-point DFTs of the even / odd samples)
template <int N, int SIGN>
__device__ __forceinline__ void dftc(float (&xr)[N], float (&xi)[N]) {
  if constexpr (N == 7) {
    float yr[7], yi[7];
    dft7c<SIGN>(xr, xi, yr, yi);
#pragma unroll
    for (int k = 0; k < 7; ++k) { xr[k] = yr[k]; xi[k] = yi[k]; }
  } else {
    float er[7], ei[7], orr[7], oi[7], Er[7], Ei[7], Or[7], Oi[7];
#pragma unroll
    for (int m = 0; m < 7; ++m) { er[m] = xr[2 * m]; ei[m] = xi[2 * m]; orr[m] = xr[2 * m + 1]; oi[m] = xi[2 * m + 1]; }
    dft7c<SIGN>(er, ei, Er, Ei);
    dft7c<SIGN>(orr, oi, Or, Oi);
#pragma unroll
    for (int k = 0; k < 7; ++k) {
      const float c = Tw<14>::c(k), s = SIGN * Tw<14>::s(k);
      const float tr = Or[k] * c - Oi[k] * s, ti = Or[k] * s + Oi[k] * c;
      xr[k] = Er[k] + tr; xi[k] = Ei[k] + ti;
      xr[k + 7] = Er[k] - tr; xi[k + 7] = Ei[k] - ti;
    }
  }
}

template <int N>
__global__ void __launch_bounds__(SCL_TPB)
gated_spectral_cl_kernel(const __nv_bfloat16* __restrict__ xz, int ld, int C,
                         const float4* __restrict__ gates, __nv_bfloat16* __restrict__ y, int ldy) {
  constexpr int Wf = N / 2 + 1, P = N * N, NB = N * Wf;
  constexpr int RH = (N + 1) / 2, KH = Wf / 2;       // rows / spectrum columns of the first thread of a plane
  constexpr float INV_N = 1.0f / (float)N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half2* R = reinterpret_cast<__half2*>(smem_raw);                      // [NB][64] (re, im)
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(R + NB * SCL_PL);   // [P][64]
  float4* gs = reinterpret_cast<float4*>(tile + P * SCL_PL);              // [NB]
  const int tid = threadIdx.x, pl = tid & (SCL_PL - 1), hf = tid / SCL_PL;
  const int slices = C / SCL_PL;
  const int n = blockIdx.x / slices, c0 = (blockIdx.x % slices) * SCL_PL;
  const __nv_bfloat16* xin = xz + (size_t)n * P * ld + c0;
  const int h_lo = hf ? RH : 0, h_hi = hf ? N : RH;
  const int k_lo = hf ? KH : 0, k_hi = hf ? Wf : KH;

  // ---- stage x tile and the sample's gate map ----
  // (asynchronous 16-byte copies: every request of the tile is in flight at once)
  for (int q = tid; q < P * 8; q += SCL_TPB) {
    const int p = q >> 3, j = q & 7;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(tile + p * SCL_PL + j * 8)),
                   "l"(xin + (size_t)p * ld + j * 8) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int i = tid; i < NB; i += SCL_TPB) gs[i] = __ldg(gates + (size_t)n * NB + i);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- forward rows: real N-point DFT -> Wf bins, scaled by 1/N ----
#pragma unroll 1
  for (int h = h_lo; h < h_hi; ++h) {
    float xv[N];
#pragma unroll
    for (int w = 0; w < N; ++w) xv[w] = __bfloat162float(tile[(h * N + w) * SCL_PL + pl]) * INV_N;
    if constexpr (N == 14) {
      // radix 2 x 7: real 7-point DFTs of the even and the odd samples (bins 0..3, the others are their
      // conjugates), X[k] = E[k mod 7] + W14^k O[k mod 7]: 110 multiply-adds per row instead of 208
      float er[4], ei[4], od[4], oi[4];
#pragma unroll
      for (int par = 0; par < 2; ++par) {
        float (&yr)[4] = par ? od : er;
        float (&yi)[4] = par ? oi : ei;
        yr[0] = xv[par]; yi[0] = 0.f;
#pragma unroll
        for (int n = 1; n < 7; ++n) yr[0] += xv[par + 2 * n];
#pragma unroll
        for (int k = 1; k < 4; ++k) {
          float ar = xv[par], ai = 0.f;
#pragma unroll
          for (int n = 1; n < 7; ++n) {
            ar = fmaf(xv[par + 2 * n], Tw<7>::c((n * k) % 7), ar);
            ai = fmaf(xv[par + 2 * n], -Tw<7>::s((n * k) % 7), ai);
          }
          yr[k] = ar; yi[k] = ai;
        }
      }
      R[(h * Wf + 0) * SCL_PL + pl] = __floats2half2_rn(er[0] + od[0], 0.f);
      R[(h * Wf + 7) * SCL_PL + pl] = __floats2half2_rn(er[0] - od[0], 0.f);
#pragma unroll
      for (int k = 1; k < 7; ++k) {
        const int kk = k <= 3 ? k : 7 - k;
        const float e_r = er[kk], e_i = k <= 3 ? ei[kk] : -ei[kk];
        const float o_r = od[kk], o_i = k <= 3 ? oi[kk] : -oi[kk];
        const float xr = fmaf(o_i, Tw<14>::s(k), fmaf(o_r, Tw<14>::c(k), e_r));
        const float xi = fmaf(-o_r, Tw<14>::s(k), fmaf(o_i, Tw<14>::c(k), e_i));
        R[(h * Wf + k) * SCL_PL + pl] = __floats2half2_rn(xr, xi);
      }
    } else {
#pragma unroll
      for (int k = 0; k < Wf; ++k) {
        float ar = xv[0], ai = 0.f;
#pragma unroll
        for (int w = 1; w < N; ++w) {
          ar = fmaf(xv[w], Tw<N>::c((w * k) % N), ar);
          ai = fmaf(xv[w], -Tw<N>::s((w * k) % N), ai);
        }
        R[(h * Wf + k) * SCL_PL + pl] = __floats2half2_rn(ar, ai);
      }
    }
  }
  __syncthreads();                      // x tile consumed; row spectra of both halves visible
  // ---- z tile (already through SiLU) into the same buffer ----
  // (asynchronous copies again: they land while the column pass runs)
  for (int q = tid; q < P * 8; q += SCL_TPB) {
    const int p = q >> 3, j = q & 7;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(tile + p * SCL_PL + j * 8)),
                   "l"(xin + C + (size_t)p * ld + j * 8) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // ---- columns: forward DFT, gates (T = 1: h = U), inverse DFT ----
#pragma unroll 1
  for (int k = k_lo; k < k_hi; ++k) {
    float vr[N], vi[N];
#pragma unroll
    for (int h = 0; h < N; ++h) {
      const float2 v = __half22float2(R[(h * Wf + k) * SCL_PL + pl]);
      vr[h] = v.x; vi[h] = v.y;
    }
    dftc<N, -1>(vr, vi);
#pragma unroll
    for (int kh = 0; kh < N; ++kh) {
      const float4 g = gs[kh * Wf + k];          // {exp(-D), (D+1e-8)B, C/(HW), 1e-7(D+1e-8)}
      const float gy = g.y * (float)N;           // undoes the row pass's 1/N
      float ur = gy * vr[kh], ui = gy * vi[kh];
      if (ur * ur + ui * ui < g.w * g.w) { ur = g.w; ui = 0.f; }
      vr[kh] = g.z * ur; vi[kh] = g.z * ui;
    }
    dftc<N, 1>(vr, vi);
#pragma unroll
    for (int h = 0; h < N; ++h) R[(h * Wf + k) * SCL_PL + pl] = __floats2half2_rn(vr[h], vi[h]);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                      // z tile complete; columns of both halves visible

  // ---- inverse rows (C2R: imaginary parts of the DC and Nyquist bins are ignored), * z ----
#pragma unroll 1
  for (int h = h_lo; h < h_hi; ++h) {
    float cr[Wf], ci[Wf];
#pragma unroll
    for (int k = 0; k < Wf; ++k) {
      const float2 v = __half22float2(R[(h * Wf + k) * SCL_PL + pl]);
      cr[k] = v.x; ci[k] = v.y;
    }
    if constexpr (N == 14) {
      // radix 2 x 7 the other way: A[k] = X[k] + conj X[7-k] gives the even samples, B[k] =
      // (X[k] - conj X[7-k]) e^{2 pi i k / 14} the odd ones, each by a real-output 7-point inverse DFT
      // from bins 0..3 (the imaginary parts of the DC and Nyquist bins do not enter)
      float a_r[4], a_i[4], b_r[4], b_i[4];
      ci[0] = 0.f; ci[7] = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float dr = cr[k] - cr[7 - k], di = ci[k] + ci[7 - k];
        a_r[k] = cr[k] + cr[7 - k]; a_i[k] = ci[k] - ci[7 - k];
        b_r[k] = dr * Tw<14>::c(k) - di * Tw<14>::s(k);
        b_i[k] = dr * Tw<14>::s(k) + di * Tw<14>::c(k);
      }
#pragma unroll
      for (int m = 0; m < 7; ++m) {
        float se = 0.f, so = 0.f;
#pragma unroll
        for (int k = 1; k < 4; ++k) {
          se = fmaf(a_r[k], Tw<7>::c((m * k) % 7), se); se = fmaf(-a_i[k], Tw<7>::s((m * k) % 7), se);
          so = fmaf(b_r[k], Tw<7>::c((m * k) % 7), so); so = fmaf(-b_i[k], Tw<7>::s((m * k) % 7), so);
        }
        const float ve = fmaf(2.f, se, a_r[0]), vo = fmaf(2.f, so, b_r[0]);
        const int idx = (h * N + 2 * m) * SCL_PL + pl;
        tile[idx] = __float2bfloat16(ve * __bfloat162float(tile[idx]));
        tile[idx + SCL_PL] = __float2bfloat16(vo * __bfloat162float(tile[idx + SCL_PL]));
      }
      continue;
    }
    constexpr int KM = (N - 1) / 2;               // bins with a conjugate partner
#pragma unroll
    for (int w = 0; w < N; ++w) {
      float acc = cr[0];
      if ((N & 1) == 0) acc += (w & 1) ? -cr[N / 2] : cr[N / 2];
      float s2 = 0.f;
#pragma unroll
      for (int k = 1; k <= KM; ++k) {
        s2 = fmaf(cr[k], Tw<N>::c((w * k) % N), s2);
        s2 = fmaf(-ci[k], Tw<N>::s((w * k) % N), s2);
      }
      acc = fmaf(2.f, s2, acc);
      const int idx = (h * N + w) * SCL_PL + pl;
      tile[idx] = __float2bfloat16(acc * __bfloat162float(tile[idx]));
    }
  }
  __syncthreads();
  __nv_bfloat16* yo = y + (size_t)n * P * ldy + c0;
  for (int q = tid; q < P * 8; q += SCL_TPB) {
    const int p = q >> 3, j = q & 7;
    *reinterpret_cast<uint4*>(yo + (size_t)p * ldy + j * 8) =
        *reinterpret_cast<const uint4*>(tile + p * SCL_PL + j * 8);
  }
}

bool spectral_cl_supported(int H, int W, int C, int T) {
  return T == 1 && H == W && (H == 14 || H == 7) && C % SCL_PL == 0;
}

// xz: (Nimg, H*W, ld) bf16 with x_main in columns [0, C) and silu(z) in [C, 2C); gates: the
// (Nimg, H*Wf) float4 maps of launch_gated_gates in row-major bin order; y: (Nimg, H*W, ldy).
int launch_gated_spectral_cl(const __nv_bfloat16* xz, int ld, int Nimg, int H, int W, int C,
                             const float* gates, __nv_bfloat16* y, int ldy, cudaStream_t st) {
  if (!spectral_cl_supported(H, W, C, 1) || ld % 8 != 0 || ldy % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  const int Wf = W / 2 + 1, NB = H * Wf, P = H * W;
  const size_t smem = (size_t)NB * SCL_PL * 4 + (size_t)P * SCL_PL * 2 + (size_t)NB * 16;
  const int grid = Nimg * (C / SCL_PL);
  cudaError_t e;
  if (H == 14) {
    e = cudaFuncSetAttribute(gated_spectral_cl_kernel<14>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    gated_spectral_cl_kernel<14><<<grid, SCL_TPB, smem, st>>>(xz, ld, C, reinterpret_cast<const float4*>(gates), y, ldy);
  } else {
    e = cudaFuncSetAttribute(gated_spectral_cl_kernel<7>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    gated_spectral_cl_kernel<7><<<grid, SCL_TPB, smem, st>>>(xz, ld, C, reinterpret_cast<const float4*>(gates), y, ldy);
  }
  return check_launch();
}

}  // namespace cssm
