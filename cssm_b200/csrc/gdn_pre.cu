// GDN block, kernels ahead of the spectral stage: RoPE + channels-last depthwise conv with
// per-row context sums, and the gate maps (alpha, beta per frequency bin; B_k, B_v per pixel).
#include "kernels.cuh"

namespace cssm {

// ------------------------------------------------- RoPE + depthwise KxK, channels-last ----
// One CTA per (frame, output row).  The K input rows are rotated (RoPE) while they are
// staged in shared memory; the conv runs from there.  The CTA also writes the sum over its
// row of the ROTATED INPUT (not of the conv output) per channel: ctx is the mean of the
// block input (cssm.py:4785-4786).
__global__ void __launch_bounds__(256)
rope_dwconv_cl_kernel(const GdnDwArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int K = a.ksz > 1 ? a.ksz : 1;
  const int lo = (K - 1) / 2;
  const int fr = blockIdx.x / a.H, h = blockIdx.x % a.H;
  const int t = fr % a.T;
  const int WC = a.W * a.C, n2 = a.C / 2;
  const int tid = threadIdx.x;
  // stage rows h-lo .. h-lo+K-1 (zeros outside the image)
  for (int r = 0; r < K; ++r) {
    const int hh = h + r - lo;
    float* dst = sm + r * WC;
    if (hh < 0 || hh >= a.H) {
      for (int i = tid; i < WC; i += blockDim.x) dst[i] = 0.f;
      continue;
    }
    const float* src = a.x + ((size_t)fr * a.H + hh) * WC;
    for (int i = tid; i < WC / 2; i += blockDim.x) {
      const int w = i / n2, pi = i % n2;
      float2 v = *reinterpret_cast<const float2*>(src + 2 * i);
      if (a.rope_t != nullptr) {
        const float2 ct = a.rope_t[t * n2 + pi], ch = a.rope_h[hh * n2 + pi], cw = a.rope_w[w * n2 + pi];
        const float cx = ct.x * ch.x - ct.y * ch.y, sx = ct.x * ch.y + ct.y * ch.x;
        const float c2 = cx * cw.x - sx * cw.y, s2 = cx * cw.y + sx * cw.x;
        v = make_float2(v.x * c2 - v.y * s2, v.x * s2 + v.y * c2);
      }
      dst[2 * i] = v.x; dst[2 * i + 1] = v.y;
    }
  }
  __syncthreads();
  // context partial sums of the centre row
  if (a.ctx_part != nullptr) {
    const float* ctr = sm + lo * WC;
    for (int c = tid; c < a.C; c += blockDim.x) {
      float s = 0.f;
      for (int w = 0; w < a.W; ++w) s += ctr[w * a.C + c];
      a.ctx_part[((size_t)fr * a.H + h) * a.C + c] = s;
    }
  }
  if (a.out != nullptr) {
    float* dst = a.out + ((size_t)fr * a.H + h) * WC;
    for (int i = tid; i < WC; i += blockDim.x) {
      const int w = i / a.C, c = i % a.C;
      float acc = a.bias[c];
      for (int r = 0; r < K; ++r)
        for (int s = 0; s < K; ++s) {
          const int ww = w + s - lo;
          if (ww < 0 || ww >= a.W) continue;
          acc = fmaf(a.wk[(size_t)(r * K + s) * a.C + c], sm[r * WC + ww * a.C + c], acc);
        }
      dst[i] = acc;
    }
  }
}

int launch_rope_dwconv_cl(const GdnDwArgs& a, cudaStream_t st) {
  const int K = a.ksz > 1 ? a.ksz : 1;
  const size_t smem = (size_t)K * a.W * a.C * sizeof(float);
  if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(rope_dwconv_cl_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  rope_dwconv_cl_kernel<<<a.BT * a.H, 256, smem, st>>>(a);
  return check_launch();
}

// ------------------------------------------------------------------- GDN gate maps ----
// One CTA per frame.  ctx = (sum over rows of ctx_part) / (H*W) + tcode[t].
// alpha/beta: sigmoid(row[h] + col[kw]) (factored) or sigmoid(Dense(H*Wf)) (dense);
// alpha = 0.1 + 0.89 * raw.  Stored as float2 {alpha, beta} at bin_index(path, kh, kw).
// B_k / B_v: same over (h, w) pixels, float2 {B_k, B_v} at h*W + w.  cssm.py:4798-4848, 4864-4865.
__global__ void __launch_bounds__(256) gdn_gates_kernel(const GdnGateArgs g) {
  extern __shared__ float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf, HW = g.H * g.W;
  float* ctx = sh;                       // [C]
  float* vec = sh + g.C;                 // factored: alpha_h, alpha_w, beta_h, beta_w, Bk_h, Bk_w, Bv_h, Bv_w
  const int fr = blockIdx.x, tid = threadIdx.x, t = fr % g.T;
  const float inv = 1.0f / (float)HW;
  for (int c = tid; c < g.C; c += blockDim.x) {
    float s = 0.f;
    for (int h = 0; h < g.H; ++h) s += g.ctx_part[((size_t)fr * g.H + h) * g.C + c];
    ctx[c] = s * inv + g.tcode[t * g.C + c];
  }
  __syncthreads();
  const int ngate = g.use_input_gates ? 4 : 2;
  if (g.gate_type == CSSM_GATE_FACTORED) {
    // segment offsets inside vec
    int off[9];
    off[0] = 0;
    for (int q = 0; q < 4; ++q) {
      const int wd = q < 2 ? Wf : g.W;
      off[2 * q + 1] = off[2 * q] + g.H;
      off[2 * q + 2] = off[2 * q + 1] + wd;
    }
    const int total = off[2 * ngate];
    for (int o = tid; o < total; o += blockDim.x) {
      int seg = 0;
      while (o >= off[seg + 1]) ++seg;
      const int col = o - off[seg];
      const int ncol = off[seg + 1] - off[seg];
      const float* kk = g.gk[seg];
      float acc = g.gb[seg][col];
      for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * ncol + col], acc);
      vec[o] = acc;
    }
    __syncthreads();
    for (int bin = tid; bin < NB; bin += blockDim.x) {
      const int kh = bin / Wf, kw = bin % Wf;
      const float ra = sigmoid_f(vec[off[0] + kh] + vec[off[1] + kw]);
      const float rb = sigmoid_f(vec[off[2] + kh] + vec[off[3] + kw]);
      g.ab[(size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf)] = make_float2(0.1f + 0.89f * ra, rb);
    }
    if (g.use_input_gates)
      for (int px = tid; px < HW; px += blockDim.x) {
        const int h = px / g.W, w = px % g.W;
        g.bkv[(size_t)fr * HW + px] = make_float2(sigmoid_f(vec[off[4] + h] + vec[off[5] + w]),
                                                  sigmoid_f(vec[off[6] + h] + vec[off[7] + w]));
      }
  } else {
    for (int bin = tid; bin < NB; bin += blockDim.x) {
      const int kh = bin / Wf, kw = bin % Wf;
      float aa = g.gb[0][bin], bb = g.gb[1][bin];
      for (int c = 0; c < g.C; ++c) {
        aa = fmaf(ctx[c], g.gk[0][(size_t)c * NB + bin], aa);
        bb = fmaf(ctx[c], g.gk[1][(size_t)c * NB + bin], bb);
      }
      g.ab[(size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf)] =
          make_float2(0.1f + 0.89f * sigmoid_f(aa), sigmoid_f(bb));
    }
    if (g.use_input_gates)
      for (int px = tid; px < HW; px += blockDim.x) {
        float aa = g.gb[2][px], bb = g.gb[3][px];
        for (int c = 0; c < g.C; ++c) {
          aa = fmaf(ctx[c], g.gk[2][(size_t)c * HW + px], aa);
          bb = fmaf(ctx[c], g.gk[3][(size_t)c * HW + px], bb);
        }
        g.bkv[(size_t)fr * HW + px] = make_float2(sigmoid_f(aa), sigmoid_f(bb));
      }
  }
}

int launch_gdn_gates(const GdnGateArgs& g, cudaStream_t st) {
  const size_t smem = (size_t)(g.C + 4 * g.H + 2 * (g.W / 2 + 1) + 2 * g.W) * sizeof(float);
  gdn_gates_kernel<<<g.BT, 256, smem, st>>>(g);
  return check_launch();
}

}  // namespace cssm
