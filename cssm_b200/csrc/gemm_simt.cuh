// fp32 CUDA-core GEMM for the 1x1 channel projections, with the layout changes and
// pointwise work of the blocks fused into its load and store:
//   A side: channels-last rows (optionally rotated by RoPE on load), or planar planes
//           (optionally RMS-normalised over channels, scaled and gated on load);
//   C side: channels-last rows, or planar planes (optionally through SiLU / sigmoid).
// out[m, n] = sum_k A[m, k] * Wk[k, n] + bias[n],  m = frame*HW + pixel.
#pragma once
#include "common.cuh"

namespace cssm {

struct GemmArgs {
  int M, N, K, HW;
  const float* A;         // channels-last: (M, K).  planar: plane (frame*a_planes + a_plane0 + k)
  int a_planes, a_plane0;
  // source frame of output frame f, both A layouts: (f / a_fdiv) * a_fmul + a_fadd, where
  // a_fdiv <= 1 means no division and a_fmul == a_fadd == 0 means the identity.
  //   last frame of every clip : a_fmul = T, a_fadd = T-1  (output frames = clips)
  //   one frame repeated over T: a_fdiv = T, a_fmul = 1    (output frames = (clip, t))
  int a_fdiv, a_fmul, a_fadd;
  int rope_tlast;         // 1: every output frame is rotated as t = T-1; 0: t = output frame % T
  const float* Wk;        // (K, N) row-major
  const float* bias;      // (N) or nullptr
  float* out;             // channels-last (M, N) or planar plane (frame*o_planes + o_plane0 + n)
  int o_planes, o_plane0;
  // RoPE on a channels-last A (nullptr = off): float2 (cos, sin) tables
  const float2* rope_t; const float2* rope_h; const float2* rope_w;
  const float* rope_nz;     // (K/2) 1 = pair is rotated, 0 = identity (may be nullptr: rotate all)
  int T, H, W;
  // planar-A prologue of the GDN output: a <- a * rsqrt(mean_k a^2 + eps) * scale[k] * gate
  const float* rms_scale;   // (K) or nullptr (no normalisation)
  const float* gate;        // planar, plane (frame*g_planes + g_plane0 + k), or nullptr
  int g_planes, g_plane0;
  int g_compact;            // 1: the gate is indexed by the OUTPUT frame, 0: by the source frame
  int out_act;              // 0 none, 1 silu, 2 sigmoid; applied to output columns n >= act_n0
  int act_n0;
  int z_last_only;          // planar output: columns n >= act_n0 are only stored for frames with t == T-1
  const float* sub;         // channels-last output only: (M, N) tensor subtracted from the result, or nullptr
};

__host__ __device__ inline int gemm_src_frame(const GemmArgs& g, int f) {
  if (g.a_fmul == 0 && g.a_fadd == 0) return f;
  return (g.a_fdiv > 1 ? f / g.a_fdiv : f) * g.a_fmul + g.a_fadd;
}
__host__ __device__ inline int gemm_rope_t(const GemmArgs& g, int f) {
  return g.rope_tlast ? g.T - 1 : f % g.T;
}

// channels-last A: source row of output row m
__host__ __device__ inline size_t gemm_src_row(const GemmArgs& g, int m) {
  if (g.a_fmul == 0 && g.a_fadd == 0) return (size_t)m;
  const int fo = m / g.HW;
  return (size_t)gemm_src_frame(g, fo) * g.HW + (m - fo * g.HW);
}

constexpr int GEMM_BM = 128, GEMM_BK = 16, GEMM_THREADS = 256;

template <int BN, bool A_PLANAR, bool O_PLANAR>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_simt_kernel(const GemmArgs g) {
  constexpr int TN = BN / 16;            // outputs per thread along n (8 or 4)
  __shared__ __align__(16) float As[GEMM_BK][GEMM_BM + 4];
  __shared__ __align__(16) float Bs[GEMM_BK][BN + 4];
  __shared__ float rinv[GEMM_BM];

  const int tid = threadIdx.x;
  // O_PLANAR: consecutive threads walk m (planes are contiguous in m); else walk n.
  const int tm = O_PLANAR ? (tid & 15) : (tid >> 4);
  const int tn = O_PLANAR ? (tid >> 4) : (tid & 15);
  const int m0 = blockIdx.x * GEMM_BM, n0 = blockIdx.y * BN;

  float acc[8][TN];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  if (A_PLANAR && g.rms_scale != nullptr) {
    // per-pixel 1/rms over all K channels of this tile's rows
    if (tid < GEMM_BM) {
      const int m = m0 + tid;
      float ss = 0.f;
      if (m < g.M) {
        const int fr = gemm_src_frame(g, m / g.HW), px = m % g.HW;
        const float* ap = g.A + ((size_t)fr * g.a_planes + g.a_plane0) * g.HW + px;
        for (int k = 0; k < g.K; ++k) { const float v = ap[(size_t)k * g.HW]; ss += v * v; }
      }
      rinv[tid] = rsqrtf(ss / (float)g.K + 1e-6f);
    }
    __syncthreads();
  }

  for (int k0 = 0; k0 < g.K; k0 += GEMM_BK) {
    // ---- A tile -> As[k][m] ----
    if (A_PLANAR) {
#pragma unroll
      for (int r = 0; r < (GEMM_BM * GEMM_BK) / GEMM_THREADS; ++r) {
        const int idx = tid + r * GEMM_THREADS;
        const int kk = idx / GEMM_BM, mm = idx % GEMM_BM;
        const int m = m0 + mm, k = k0 + kk;
        float v = 0.f;
        if (m < g.M && k < g.K) {
          const int fr = gemm_src_frame(g, m / g.HW), px = m % g.HW;
          v = g.A[((size_t)fr * g.a_planes + g.a_plane0 + k) * g.HW + px];
          if (g.rms_scale != nullptr) v *= rinv[mm] * g.rms_scale[k];
          if (g.gate != nullptr) {
            const int fg = g.g_compact ? m / g.HW : fr;
            v *= g.gate[((size_t)fg * g.g_planes + g.g_plane0 + k) * g.HW + px];
          }
        }
        As[kk][mm] = v;
      }
    } else {
#pragma unroll
      for (int r = 0; r < (GEMM_BM * GEMM_BK / 4) / GEMM_THREADS; ++r) {
        const int idx = tid + r * GEMM_THREADS;
        const int mm = idx >> 2, kq = (idx & 3) * 4;
        const int m = m0 + mm, k = k0 + kq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < g.M && k < g.K) {
          v = *reinterpret_cast<const float4*>(g.A + gemm_src_row(g, m) * g.K + k);
          if (g.rope_t != nullptr) {
            const int px = m % g.HW;
            const int t = gemm_rope_t(g, m / g.HW), h = px / g.W, w = px % g.W;
            const int n2 = g.K >> 1, i = k >> 1;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float2 ct = g.rope_t[t * n2 + i + e];
              const float2 ch = g.rope_h[h * n2 + i + e];
              const float2 cw = g.rope_w[w * n2 + i + e];
              // (cos, sin) of the summed angle
              float cx = ct.x * ch.x - ct.y * ch.y, sx = ct.x * ch.y + ct.y * ch.x;
              const float c2 = cx * cw.x - sx * cw.y, s2 = cx * cw.y + sx * cw.x;
              float& xe = e ? v.z : v.x;
              float& xo = e ? v.w : v.y;
              const float ne = xe * c2 - xo * s2, no = xe * s2 + xo * c2;
              xe = ne; xo = no;
            }
          }
        }
        As[kq + 0][mm] = v.x; As[kq + 1][mm] = v.y; As[kq + 2][mm] = v.z; As[kq + 3][mm] = v.w;
      }
    }
    // ---- W tile -> Bs[k][n] ----
    for (int idx = tid; idx < GEMM_BK * BN; idx += GEMM_THREADS) {
      const int kk = idx / BN, nn = idx % BN;
      const int k = k0 + kk, n = n0 + nn;
      Bs[kk][nn] = (k < g.K && n < g.N) ? g.Wk[(size_t)k * g.N + n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GEMM_BK; ++kk) {
      float av[8], bv[TN];
      const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][tm * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + tm * 4]);
      av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
      av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[kk][tn * 4]);
      bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
      if (TN == 8) {
        const float4 b1 = *reinterpret_cast<const float4*>(&Bs[kk][BN / 2 + tn * 4]);
        bv[TN - 4] = b1.x; bv[TN - 3] = b1.y; bv[TN - 2] = b1.z; bv[TN - 1] = b1.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

  // ---- epilogue ----
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? tm * 4 + i : 64 + tm * 4 + (i - 4));
    if (m >= g.M) continue;
    const int fr = m / g.HW, px = m % g.HW;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + (j < 4 ? tn * 4 + j : BN / 2 + tn * 4 + (j - 4));
      if (n >= g.N) continue;
      float v = acc[i][j] + (g.bias ? g.bias[n] : 0.f);
      if (n >= g.act_n0) {
        if (g.out_act == 1) v = silu_f(v);
        else if (g.out_act == 2) v = sigmoid_f(v);
      }
      if (O_PLANAR) {
        if (g.z_last_only && n >= g.act_n0 && fr % g.T != g.T - 1) continue;
        g.out[((size_t)fr * g.o_planes + g.o_plane0 + n) * g.HW + px] = v;
      }
      else g.out[(size_t)m * g.N + n] = g.sub ? v - g.sub[(size_t)m * g.N + n] : v;
    }
  }
}

template <bool A_PLANAR, bool O_PLANAR>
inline int launch_gemm_simt(const GemmArgs& g, cudaStream_t st) {
  const dim3 block(GEMM_THREADS);
  if (g.N > 64) {
    const dim3 grid((g.M + GEMM_BM - 1) / GEMM_BM, (g.N + 127) / 128);
    gemm_simt_kernel<128, A_PLANAR, O_PLANAR><<<grid, block, 0, st>>>(g);
  } else {
    const dim3 grid((g.M + GEMM_BM - 1) / GEMM_BM, 1);
    gemm_simt_kernel<64, A_PLANAR, O_PLANAR><<<grid, block, 0, st>>>(g);
  }
  return check_launch();
}

// Tensor-core (tcgen05) variant for K = 64, N in {64, 128}, H*W a multiple of 128.
bool gemm_tc_supported(const GemmArgs& g, bool a_planar);
int launch_gemm_tc(const GemmArgs& g, bool a_planar, cudaStream_t st);
int read_tc_error(int* out);

// Picks the tensor-core kernel when it covers the problem, else the CUDA-core kernel.
template <bool A_PLANAR, bool O_PLANAR>
inline int launch_gemm(const GemmArgs& g, cudaStream_t st) {
  static_assert(A_PLANAR != O_PLANAR, "projections change layout");
  if (gemm_tc_supported(g, A_PLANAR)) return launch_gemm_tc(g, A_PLANAR, st);
  return launch_gemm_simt<A_PLANAR, O_PLANAR>(g, st);
}

}  // namespace cssm
