// extern "C" entry points of the DeltaNetCSSM block (src/models/cssm.py:3628-3930): the scalar
// delta rule per channel and frequency bin,
//   A_t = squash(alpha_t W_hat (1 - beta_t |k_t|^2)),  U_t = beta_t v_t conj(k_t),
//   h_t = A_t h_{t-1} + U_t,  o_t = h_t q_t,
// with q and k L2-normalised over the half-spectrum of their plane.  One CTA per (batch, channel)
// walks t = 0..T-1 with the state h in shared memory; the transforms are the direct-DFT plane
// routines (any H, W).  A_t and U_t are never materialised.
#include <string.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"
#include "generic_dft.cuh"

namespace cssm {

struct DnGateArgs {
  const float* ctx_part; const float* tcode;   // (BT,H,C) row sums of the rotated input, (T,C)
  int BT, T, C, H, W, gate_type, path;
  const float* gk[10]; const float* gb[10];    // alpha, beta, B_k, B_v, C_gate (x {h, w} if factored)
  float4* abkv;                                // (BT, H*Wf) {alpha, beta, B_k, B_v} at bin_index(path, ...)
  float* cg;                                   // (BT, H*Wf) C_gate / (H*W)
};

__device__ __forceinline__ float dn_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// One CTA per (frame, chunk of bins): ctx = mean of the rotated input + temporal code, then the
// five gate maps sigmoid(Dense(ctx)) (dense) or sigmoid(row + col) (factored); alpha is mapped
// to [0.1, 0.99] (cssm.py:3756-3793).
__global__ void __launch_bounds__(256) deltanet_gates_kernel(const DnGateArgs g) {
  extern __shared__ float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf;
  float* ctx = sh;                 // [C]
  float* vec = sh + g.C;           // factored: 5 x (H + Wf)
  const int fr = blockIdx.x, tid = threadIdx.x, t = fr % g.T;
  const float inv = 1.0f / (float)(g.H * g.W);
  for (int c = tid; c < g.C; c += blockDim.x) {
    float s = 0.f;
    for (int h = 0; h < g.H; ++h) s += g.ctx_part[((size_t)fr * g.H + h) * g.C + c];
    ctx[c] = s * inv + g.tcode[t * g.C + c];
  }
  __syncthreads();
  const int per = g.H + Wf;
  if (g.gate_type == CSSM_GATE_FACTORED) {
    for (int o = tid; o < 5 * per; o += blockDim.x) {
      const int gi = o / per, r = o % per;
      const bool isw = r >= g.H;
      const int col = isw ? r - g.H : r, ncol = isw ? Wf : g.H;
      const float* kk = g.gk[2 * gi + (isw ? 1 : 0)];
      float acc = g.gb[2 * gi + (isw ? 1 : 0)][col];
      for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * ncol + col], acc);
      vec[o] = acc;
    }
    __syncthreads();
  }
  const int per_cta = (NB + gridDim.y - 1) / gridDim.y;
  const int bin_end = min(NB, (int)(blockIdx.y + 1) * per_cta);
  for (int bin = blockIdx.y * per_cta + tid; bin < bin_end; bin += blockDim.x) {
    const int kh = bin / Wf, kw = bin % Wf;
    float r[5];
    if (g.gate_type == CSSM_GATE_FACTORED) {
#pragma unroll
      for (int gi = 0; gi < 5; ++gi) r[gi] = vec[gi * per + kh] + vec[gi * per + g.H + kw];
    } else {
#pragma unroll
      for (int gi = 0; gi < 5; ++gi) {
        float acc = g.gb[gi][bin];
        const float* kk = g.gk[gi];
        for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * NB + bin], acc);
        r[gi] = acc;
      }
    }
    const size_t oi = (size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf);
    g.abkv[oi] = make_float4(0.1f + 0.89f * dn_sigmoid(r[0]), dn_sigmoid(r[1]),
                                                dn_sigmoid(r[2]), dn_sigmoid(r[3]));
    g.cg[oi] = dn_sigmoid(r[4]) * inv;
  }
}

__global__ void __launch_bounds__(GG_THREADS) deltanet_spectral_kernel(const DnSpectralArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.H, W = a.W;
  const int Wf = W / 2 + 1, HW = H * W, NB = H * Wf;
  float* xs = reinterpret_cast<float*>(smem_raw);
  cf* twW = reinterpret_cast<cf*>(xs + ((HW + 1) & ~1));
  cf* twH = twW + W;
  cf* Rb = twH + H;
  cf* SQ = Rb + NB;      // query spectrum
  cf* SK = SQ + NB;      // gated key spectrum
  cf* Fb = SK + NB;      // gated value spectrum, then the output spectrum
  cf* hst = Fb + NB;     // state
  __shared__ float red[GG_THREADS / 32];

  const int tid = threadIdx.x;
  const int b = blockIdx.x / a.C, ch = blockIdx.x % a.C;
  for (int i = tid; i < W; i += GG_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)W, &s, &co); twW[i] = mk(co, s);
  }
  for (int i = tid; i < H; i += GG_THREADS) {
    float s, co; sincospif(-2.0f * (float)i / (float)H, &s, &co); twH[i] = mk(co, s);
  }
  for (int o = tid; o < NB; o += GG_THREADS) hst[o] = mk(0.f, 0.f);
  const cf* wh = a.what + (size_t)ch * NB;
  const float floor_mag = a.goom_floor ? 1e-7f : 0.f;

  for (int t = 0; t < a.T; ++t) {
    const size_t frame = (size_t)(b * a.T + t);
    float* base = a.qkv + frame * 3 * a.C * HW;
    const float4* gm = a.abkv + frame * NB;
    const float* cg = a.cg + frame * NB;
    const bool chan = a.chan != nullptr;
    const float2 ab = chan ? a.chan[frame * a.C + ch] : make_float2(0.f, 0.f);
    const float invHW = 1.0f / (float)HW;
    // q: spectrum and its L2 norm over the half-spectrum bins
    gen_fwd_plane(base + (size_t)ch * HW, xs, Rb, SQ, twW, twH, H, W);
    float p = 0.f;
    for (int o = tid; o < NB; o += GG_THREADS) { const cf z = SQ[o]; p += z.x * z.x + z.y * z.y; }
    const float nq = rsqrtf(block_sum(p, red) + 1e-6f);
    // k: spectrum times B_k, then its norm
    gen_fwd_plane(base + (size_t)(a.C + ch) * HW, xs, Rb, SK, twW, twH, H, W);
    p = 0.f;
    for (int o = tid; o < NB; o += GG_THREADS) {
      const float bk = chan ? 1.f : gm[o].z;
      const cf z = mk(SK[o].x * bk, SK[o].y * bk);
      SK[o] = z;
      p += z.x * z.x + z.y * z.y;
    }
    const float nk = rsqrtf(block_sum(p, red) + 1e-6f);
    // v
    float* vplane = base + (size_t)(2 * a.C + ch) * HW;
    gen_fwd_plane(vplane, xs, Rb, Fb, twW, twH, H, W);
    // per-bin delta rule (each thread owns its bins)
    for (int o = tid; o < NB; o += GG_THREADS) {
      const float4 g = chan ? make_float4(ab.x, ab.y, 1.f, 1.f) : gm[o];
      const cf k = mk(SK[o].x * nk, SK[o].y * nk);
      const cf q = mk(SQ[o].x * nq, SQ[o].y * nq);
      const cf v = mk(Fb[o].x * g.w, Fb[o].y * g.w);
      const float kp = k.x * k.x + k.y * k.y;
      const float sc = g.x * (1.0f - g.y * kp);
      cf A = mk(wh[o].x * sc, wh[o].y * sc);
      const float am = sqrtf(A.x * A.x + A.y * A.y);
      const float sq = a.rho / (1.0f + am);
      A = mk(A.x * sq, A.y * sq);
      if (am * sq < floor_mag) A = mk(floor_mag, 0.f);
      cf U = cmulc(v, k);                      // v * conj(k)
      U = mk(U.x * g.y, U.y * g.y);
      if (U.x * U.x + U.y * U.y < floor_mag * floor_mag) U = mk(floor_mag, 0.f);
      cf h = cmul(A, hst[o]);
      h.x += U.x; h.y += U.y;
      hst[o] = h;
      const cf oq = cmul(h, q);
      const float c = chan ? invHW : cg[o];
      Fb[o] = mk(oq.x * c, oq.y * c);
    }
    gen_inv_plane(Fb, Rb, vplane, twW, twH, H, W);
  }
}

// gate_type 'channel': alpha, beta = per-channel scalars from Dense(C)(ctx) (cssm.py:3764-3768).
// One CTA per frame.
struct DnChanArgs {
  const float* ctx_part; const float* tcode;
  int BT, T, C, H, W;
  const float* ak; const float* ab; const float* bk; const float* bb;   // (C,C), (C) x 2
  float2* chan;                                                          // (BT, C) {alpha, beta}
};
__global__ void __launch_bounds__(128) deltanet_chan_gates_kernel(const DnChanArgs g) {
  extern __shared__ float sh[];          // ctx [C]
  const int fr = blockIdx.x, tid = threadIdx.x, t = fr % g.T;
  const float inv = 1.0f / (float)(g.H * g.W);
  for (int c = tid; c < g.C; c += blockDim.x) {
    float s = 0.f;
    for (int h = 0; h < g.H; ++h) s += g.ctx_part[((size_t)fr * g.H + h) * g.C + c];
    sh[c] = s * inv + g.tcode[t * g.C + c];
  }
  __syncthreads();
  for (int o = tid; o < g.C; o += blockDim.x) {
    float aa = g.ab[o], bb = g.bb[o];
    for (int c = 0; c < g.C; ++c) {
      aa = fmaf(sh[c], g.ak[(size_t)c * g.C + o], aa);
      bb = fmaf(sh[c], g.bk[(size_t)c * g.C + o], bb);
    }
    g.chan[(size_t)fr * g.C + o] = make_float2(0.1f + 0.89f * dn_sigmoid(aa), dn_sigmoid(bb));
  }
}

// k, v planes times their spatial gate planes: for every frame the 2C planes C..3C of the
// (frames, 3C, HW) q/k/v buffer are multiplied by planes 0..2C of the (frames, 3C, HW) gate buffer
__global__ void __launch_bounds__(256) deltanet_kv_gate_kernel(float* __restrict__ qkv,
                                                               const float* __restrict__ gsp,
                                                               size_t per_frame4, size_t fstride4,
                                                               size_t total4, size_t koff4) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total4) return;
  const size_t fr = i / per_frame4, r = i - fr * per_frame4;
  float4* d = reinterpret_cast<float4*>(qkv) + fr * fstride4 + koff4 + r;
  const float4 gv = __ldg(reinterpret_cast<const float4*>(gsp) + fr * fstride4 + r);
  float4 v = *d;
  v.x *= gv.x; v.y *= gv.y; v.z *= gv.z; v.w *= gv.w;
  *d = v;
}

static size_t deltanet_smem_bytes(int H, int W) {
  const size_t Wf = W / 2 + 1, NB = (size_t)H * Wf;
  const size_t fl = ((size_t)H * W + 1) & ~(size_t)1;
  return fl * 4 + (W + H + 5 * NB) * sizeof(cf);
}

static int deltanet_path(const cssm_deltanet_desc& d) {
  const SpectralPath p = spectral_path(d.H, d.W);
  return (p == PATH_R64 || p == PATH_R32) ? p : PATH_GENERIC;
}

static int deltanet_validate(const cssm_deltanet_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->kernel_size <= 0)
    return CSSM_ERR_DIMS;
  if (d->goom_floor != 0 && d->goom_floor != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (d->rope_mode < CSSM_ROPE_NONE || d->rope_mode > CSSM_ROPE_MROPE) return CSSM_ERR_UNSUPPORTED;
  if (d->gate_type != CSSM_GATE_DENSE && d->gate_type != CSSM_GATE_FACTORED &&
      d->gate_type != CSSM_GATE_CHANNEL)
    return CSSM_ERR_UNSUPPORTED;
  const bool crop_h = d->kernel_size > d->H, crop_w = d->kernel_size > d->W;
  if (crop_h != crop_w) return CSSM_ERR_UNSUPPORTED;
  if (deltanet_smem_bytes(d->H, d->W) > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

struct DnPlan { size_t what, rope_t, rope_h, rope_w, rope_nz, tcode, gw, gb, total; };
static DnPlan deltanet_plan_layout(const cssm_deltanet_desc& d) {
  DnPlan p;
  const size_t Wf = d.W / 2 + 1, n2 = d.C / 2;
  size_t off = 0;
  p.what = off;   off += round_up((size_t)d.C * d.H * Wf * sizeof(cf), 256);
  p.rope_t = off; off += round_up((size_t)d.T * n2 * sizeof(float2), 256);
  p.rope_h = off; off += round_up((size_t)d.H * n2 * sizeof(float2), 256);
  p.rope_w = off; off += round_up((size_t)d.W * n2 * sizeof(float2), 256);
  p.rope_nz = off; off += round_up(n2 * sizeof(float), 256);
  p.tcode = off;  off += round_up((size_t)d.T * d.C * sizeof(float), 256);
  // channel gates: the B_k, B_v, C_gate conv kernels packed side by side as one (C, 3C) matrix
  const bool ch = d.gate_type == CSSM_GATE_CHANNEL;
  p.gw = off;     off += ch ? round_up((size_t)d.C * 3 * d.C * sizeof(float), 256) : 0;
  p.gb = off;     off += ch ? round_up((size_t)3 * d.C * sizeof(float), 256) : 0;
  p.total = off;
  return p;
}

struct DnWs { size_t qkv, ctx_part, abkv, cg, gsp, chan, total; };
static DnWs deltanet_ws_layout(const cssm_deltanet_desc& d) {
  DnWs l;
  const size_t BT = (size_t)d.B * d.T, HW = (size_t)d.H * d.W, NB = (size_t)d.H * (d.W / 2 + 1);
  size_t off = 0;
  l.qkv = off;      off += round_up(BT * 3 * d.C * HW * sizeof(float), 256);
  l.ctx_part = off; off += round_up(BT * d.H * d.C * sizeof(float), 256);
  l.abkv = off;     off += round_up(BT * NB * sizeof(float4), 256);
  l.cg = off;       off += round_up(BT * NB * sizeof(float), 256);
  const bool ch = d.gate_type == CSSM_GATE_CHANNEL;
  l.gsp = off;      off += ch ? round_up(BT * 3 * d.C * HW * sizeof(float), 256) : 0;   // B_k, B_v, C_gate planes
  l.chan = off;     off += ch ? round_up(BT * d.C * sizeof(float2), 256) : 0;
  l.total = off;
  return l;
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_deltanet_plan_bytes(const cssm_deltanet_desc* d) {
  return deltanet_validate(d) == CSSM_OK ? deltanet_plan_layout(*d).total : 0;
}

size_t cssm_deltanet_workspace_bytes(const cssm_deltanet_desc* d) {
  return deltanet_validate(d) == CSSM_OK ? deltanet_ws_layout(*d).total : 0;
}

int cssm_deltanet_plan_init(const cssm_deltanet_desc* d, const cssm_deltanet_weights* w, void* plan,
                            size_t plan_bytes, void* stream) {
  int s = deltanet_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->kernel || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  const DnPlan p = deltanet_plan_layout(*d);
  if (plan_bytes < p.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = (char*)plan;
  // W_hat is squashed but not floored: the floor of the log-space scan acts on A_t and U_t
  s = launch_khat(w->kernel, (cf*)(base + p.what), d->C, d->kernel_size, d->H, d->W,
                  d->spectral_rho, 1, 0, deltanet_path(*d), st);
  if (s != CSSM_OK) return s;
  s = launch_rope_tables((float2*)(base + p.rope_t), (float2*)(base + p.rope_h),
                         (float2*)(base + p.rope_w), (float*)(base + p.rope_nz), d->T, d->H, d->W,
                         d->C, d->rope_mode, d->rope_base, st);
  if (s != CSSM_OK) return s;
  if (d->gate_type == CSSM_GATE_CHANNEL) {
    const size_t cb = (size_t)d->C * sizeof(float);
    for (int i = 0; i < 3; ++i) {
      if (!w->gate_kernel[2 + i] || !w->gate_bias[2 + i]) return CSSM_ERR_NULL;
      cudaError_t e = cudaMemcpy2DAsync(base + p.gw + i * cb, 3 * cb, w->gate_kernel[2 + i], cb, cb,
                                        (size_t)d->C, cudaMemcpyDeviceToDevice, st);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(base + p.gb + i * cb, w->gate_bias[2 + i], cb, cudaMemcpyDeviceToDevice, st);
      if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    }
  }
  return launch_tcode((float*)(base + p.tcode), d->T, d->C, d->rope_base, st);
}

int cssm_deltanet_forward(const cssm_deltanet_desc* d, const cssm_deltanet_weights* w,
                          const void* plan, const float* x, float* y, void* workspace,
                          size_t workspace_bytes, void* stream) {
  int s = deltanet_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan || !x || !y || !workspace) return CSSM_ERR_NULL;
  if (!w->qkv_proj_kernel || !w->qkv_proj_bias || !w->output_proj_kernel || !w->output_proj_bias)
    return CSSM_ERR_NULL;
  const bool chan = d->gate_type == CSSM_GATE_CHANNEL;
  const int nptr = d->gate_type == CSSM_GATE_FACTORED ? 10 : 5;
  for (int i = 0; i < nptr; ++i)
    if (!w->gate_kernel[i] || !w->gate_bias[i]) return CSSM_ERR_NULL;
  if (!aligned16(x) || !aligned16(y) || !aligned16(plan) || !aligned16(workspace))
    return CSSM_ERR_ALIGN;
  const DnWs l = deltanet_ws_layout(*d);
  if (workspace_bytes < l.total) return CSSM_ERR_WORKSPACE;
  const DnPlan p = deltanet_plan_layout(*d);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  const char* pl = (const char*)plan;
  const int BT = d->B * d->T, HW = d->H * d->W, C = d->C;
  const bool rope = d->rope_mode != CSSM_ROPE_NONE;
  const float2* rt = rope ? (const float2*)(pl + p.rope_t) : nullptr;
  const float2* rh = rope ? (const float2*)(pl + p.rope_h) : nullptr;
  const float2* rw = rope ? (const float2*)(pl + p.rope_w) : nullptr;
  const float* rnz = rope ? (const float*)(pl + p.rope_nz) : nullptr;
  float* qkv = (float*)(ws + l.qkv);

  // 1. context row sums of the rotated input
  GdnDwArgs dw;
  memset(&dw, 0, sizeof(dw));
  dw.x = x; dw.out = nullptr; dw.ksz = 1;
  dw.BT = BT; dw.T = d->T; dw.H = d->H; dw.W = d->W; dw.C = C;
  dw.rope_t = rt; dw.rope_h = rh; dw.rope_w = rw;
  dw.ctx_part = (float*)(ws + l.ctx_part);
  if ((s = launch_rope_dwconv_cl(dw, st)) != CSSM_OK) return s;

  // 2. qkv projection of the rotated input -> planar (BT, 3C, H, W)
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = BT * HW; g.N = 3 * C; g.K = C; g.HW = HW;
  g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
  g.Wk = w->qkv_proj_kernel; g.bias = w->qkv_proj_bias;
  g.out = qkv; g.o_planes = 3 * C; g.o_plane0 = 0;
  g.T = d->T; g.H = d->H; g.W = d->W;
  if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;

  // 3. gate maps (dense / factored) or channel gates
  DnGateArgs ga;
  memset(&ga, 0, sizeof(ga));
  ga.ctx_part = dw.ctx_part; ga.tcode = (const float*)(pl + p.tcode);
  ga.BT = BT; ga.T = d->T; ga.C = C; ga.H = d->H; ga.W = d->W; ga.gate_type = d->gate_type;
  ga.path = deltanet_path(*d);
  for (int i = 0; i < nptr; ++i) { ga.gk[i] = w->gate_kernel[i]; ga.gb[i] = w->gate_bias[i]; }
  ga.abkv = (float4*)(ws + l.abkv); ga.cg = (float*)(ws + l.cg);
  if (chan) {
    DnChanArgs ca;
    memset(&ca, 0, sizeof(ca));
    ca.ctx_part = dw.ctx_part; ca.tcode = ga.tcode;
    ca.BT = BT; ca.T = d->T; ca.C = C; ca.H = d->H; ca.W = d->W;
    ca.ak = w->gate_kernel[0]; ca.ab = w->gate_bias[0]; ca.bk = w->gate_kernel[1]; ca.bb = w->gate_bias[1];
    ca.chan = (float2*)(ws + l.chan);
    deltanet_chan_gates_kernel<<<BT, 128, (size_t)C * sizeof(float), st>>>(ca);
    if ((s = check_launch()) != CSSM_OK) return s;
    // spatial gates sigmoid(Conv1x1(rotated x)) -> planes (BT, 3C, H, W): B_k, B_v, C_gate
    float* gsp = (float*)(ws + l.gsp);
    memset(&g, 0, sizeof(g));
    g.M = BT * HW; g.N = 3 * C; g.K = C; g.HW = HW;
    g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
    g.Wk = (const float*)(pl + p.gw); g.bias = (const float*)(pl + p.gb);     // packed by plan_init
    g.out = gsp; g.o_planes = 3 * C; g.o_plane0 = 0;
    g.T = d->T; g.H = d->H; g.W = d->W;
    g.out_act = 2; g.act_n0 = 0;
    if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;
    // k *= B_k, v *= B_v in the spatial domain
    // C is a multiple of 4, so every frame's planes start and end on a float4 boundary
    const size_t per_frame4 = (size_t)2 * C * HW / 4, fstride4 = (size_t)3 * C * HW / 4;
    const size_t total4 = per_frame4 * BT;
    deltanet_kv_gate_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, st>>>(
        qkv, gsp, per_frame4, fstride4, total4, (size_t)C * HW / 4);
    if ((s = check_launch()) != CSSM_OK) return s;
  } else {
    const int Wf = d->W / 2 + 1, NB = d->H * Wf;
    const size_t smem = (size_t)(C + 5 * (d->H + Wf)) * sizeof(float);
    int chunks = 1;
    if (BT < 296) {
      chunks = (296 + BT - 1) / BT;
      const int maxc = (NB + 255) / 256;
      if (chunks > maxc) chunks = maxc;
    }
    deltanet_gates_kernel<<<dim3(BT, chunks), 256, smem, st>>>(ga);
    if ((s = check_launch()) != CSSM_OK) return s;
  }

  // 4. fused transforms + delta rule + output gate, output planes over the v planes
  DnSpectralArgs sp;
  memset(&sp, 0, sizeof(sp));
  sp.qkv = qkv; sp.what = (const cf*)(pl + p.what); sp.abkv = ga.abkv; sp.cg = ga.cg;
  sp.B = d->B; sp.T = d->T; sp.C = C; sp.H = d->H; sp.W = d->W;
  sp.rho = d->spectral_rho; sp.goom_floor = d->goom_floor;
  sp.chan = chan ? (const float2*)(ws + l.chan) : nullptr;
  if (deltanet_path(*d) == PATH_R64) {
    if ((s = launch_deltanet_spectral_r64(sp, st)) != CSSM_OK) return s;
  } else if (deltanet_path(*d) == PATH_R32) {
    if ((s = launch_deltanet_spectral_r32(sp, st)) != CSSM_OK) return s;
  } else {
    const size_t smem = deltanet_smem_bytes(d->H, d->W);
    cudaError_t e = cudaFuncSetAttribute(deltanet_spectral_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    deltanet_spectral_kernel<<<d->B * C, GG_THREADS, smem, st>>>(sp);
    if ((s = check_launch()) != CSSM_OK) return s;
  }

  // 5. output_proj of the output planes -> channels-last y
  memset(&g, 0, sizeof(g));
  g.M = BT * HW; g.N = C; g.K = C; g.HW = HW;
  g.A = qkv; g.a_planes = 3 * C; g.a_plane0 = 2 * C;
  if (chan) { g.gate = (const float*)(ws + l.gsp); g.g_planes = 3 * C; g.g_plane0 = 2 * C; }   // * C_gate
  g.Wk = w->output_proj_kernel; g.bias = w->output_proj_bias;
  g.out = y;
  g.T = d->T; g.H = d->H; g.W = d->W;
  return launch_gemm<true, false>(g, st);
}

}  // extern "C"
