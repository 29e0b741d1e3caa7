// extern "C" entry points of the single-state AdditiveCSSM block (single_state=True,
// src/models/cssm.py:2961-3359, 3580-3626):
//   RoPE -> Dense x_proj -> rfft2 -> h_t = (d_X K_hat) h_{t-1} + B_X X_hat_t -> C_gate h_t -> irfft2
//   -> Dense output_proj,
// with the three gate maps computed from the spatial mean of the rotated input plus the temporal
// code.  The recurrence runs in the gated block's fused spectral kernels (mode 2: gate maps, no
// z planes); this file adds the gate-map kernel and the sequencing.
#include <string.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"

namespace cssm {

struct AddGateArgs {
  const float* ctx_part; const float* tcode;   // (BT,H,C) row sums of the rotated input, (T,C)
  int BT, T, C, H, W, gate_type, path, goom_floor;
  const float* gk[6]; const float* gb[6];
  float4* maps;                                // (BT, H*Wf) in spectral bin order
};

__device__ __forceinline__ float add_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// One CTA per (frame, chunk of bins).  The map entry has the layout the fused spectral kernel
// reads: {factor on K_hat, factor on X_hat, factor on the state for the output (with the 1/(HW)
// of the inverse transform folded in), magnitude floor of the input term}.
__global__ void __launch_bounds__(256) additive_gates_kernel(const AddGateArgs g) {
  extern __shared__ float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf;
  float* ctx = sh;                 // [C]
  float* vec = sh + g.C;           // factored: 3 x (H + Wf)
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
    for (int o = tid; o < 3 * per; o += blockDim.x) {
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
    float r[3];
    if (g.gate_type == CSSM_GATE_FACTORED) {
#pragma unroll
      for (int gi = 0; gi < 3; ++gi) r[gi] = vec[gi * per + kh] + vec[gi * per + g.H + kw];
    } else {
#pragma unroll
      for (int gi = 0; gi < 3; ++gi) {
        float acc = g.gb[gi][bin];
        const float* kk = g.gk[gi];
        for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * NB + bin], acc);
        r[gi] = acc;
      }
    }
    float4 o;
    o.x = 0.1f + 0.89f * add_sigmoid(r[0]);
    o.y = add_sigmoid(r[1]);
    o.z = add_sigmoid(r[2]) * inv;
    o.w = g.goom_floor ? 1e-7f : 0.f;
    g.maps[(size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf)] = o;
  }
}

// gate_type 'channel' (cssm.py:3168-3178): d_X = 0.1 + 0.89 sigmoid(Dense(C)(ctx)) per (frame,
// channel); B_X and C_gate are per-pixel maps sigmoid(Conv1x1(rotated x)) applied in the spatial
// domain, so the per-bin maps are the constants {1, 1, 1/(HW), floor}.  One CTA per frame.
struct AddChanArgs {
  const float* ctx_part; const float* tcode;
  int BT, T, C, H, W, goom_floor;
  const float* dk; const float* db;        // (C, C), (C)
  float* dchan;                            // (BT, C)
  float4* maps;                            // (BT, H*Wf)
};
__global__ void __launch_bounds__(128) additive_chan_gates_kernel(const AddChanArgs g) {
  extern __shared__ float sh[];            // ctx [C]
  const int fr = blockIdx.x, tid = threadIdx.x, t = fr % g.T;
  const int NB = g.H * (g.W / 2 + 1);
  const float inv = 1.0f / (float)(g.H * g.W);
  for (int c = tid; c < g.C; c += blockDim.x) {
    float s = 0.f;
    for (int h = 0; h < g.H; ++h) s += g.ctx_part[((size_t)fr * g.H + h) * g.C + c];
    sh[c] = s * inv + g.tcode[t * g.C + c];
  }
  __syncthreads();
  for (int o = tid; o < g.C; o += blockDim.x) {
    float a = g.db[o];
    for (int c = 0; c < g.C; ++c) a = fmaf(sh[c], g.dk[(size_t)c * g.C + o], a);
    g.dchan[(size_t)fr * g.C + o] = 0.1f + 0.89f * add_sigmoid(a);
  }
  const float4 m = make_float4(1.f, 1.f, inv, g.goom_floor ? 1e-7f : 0.f);
  for (int i = tid; i < NB; i += blockDim.x) g.maps[(size_t)fr * NB + i] = m;
}

// planes [0, C) of every frame of the (frames, 2C, HW) buffer times its planes [C, 2C)
__global__ void __launch_bounds__(256) additive_in_gate_kernel(float* __restrict__ planar, size_t per_frame4,
                                                               size_t total4) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total4) return;
  const size_t fr = i / per_frame4, r = i - fr * per_frame4;
  float4* d = reinterpret_cast<float4*>(planar) + fr * 2 * per_frame4 + r;
  const float4 gv = d[per_frame4];
  float4 v = *d;
  v.x *= gv.x; v.y *= gv.y; v.z *= gv.z; v.w *= gv.w;
  *d = v;
}

static int launch_additive_gates(const AddGateArgs& g, cudaStream_t st) {
  const int Wf = g.W / 2 + 1, NB = g.H * Wf;
  const size_t smem = (size_t)(g.C + 3 * (g.H + Wf)) * sizeof(float);
  int chunks = 1;
  if (g.BT < 296) {
    chunks = (296 + g.BT - 1) / g.BT;
    const int maxc = (NB + 255) / 256;
    if (chunks > maxc) chunks = maxc;
  }
  additive_gates_kernel<<<dim3(g.BT, chunks), 256, smem, st>>>(g);
  return check_launch();
}

static int additive_validate(const cssm_additive_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->kernel_size <= 0)
    return CSSM_ERR_DIMS;
  if (d->single_state != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->goom_floor != 0 && d->goom_floor != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (d->rope_mode < CSSM_ROPE_NONE || d->rope_mode > CSSM_ROPE_MROPE) return CSSM_ERR_UNSUPPORTED;
  if (d->gate_type != CSSM_GATE_DENSE && d->gate_type != CSSM_GATE_FACTORED &&
      d->gate_type != CSSM_GATE_CHANNEL)
    return CSSM_ERR_UNSUPPORTED;
  const bool crop_h = d->kernel_size > d->H, crop_w = d->kernel_size > d->W;
  if (crop_h != crop_w) return CSSM_ERR_UNSUPPORTED;
  if (spectral_path(d->H, d->W) == PATH_GENERIC && generic_smem_bytes(d->H, d->W) > 200 * 1024)
    return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

struct AddPlan { size_t khat, rope_t, rope_h, rope_w, rope_nz, tcode, gw, gb, total; };
static AddPlan additive_plan_layout(const cssm_additive_desc& d) {
  AddPlan p;
  const size_t Wf = d.W / 2 + 1, n2 = d.C / 2;
  size_t off = 0;
  p.khat = off;   off += round_up((size_t)d.C * d.H * Wf * sizeof(cf), 256);
  p.rope_t = off; off += round_up((size_t)d.T * n2 * sizeof(float2), 256);
  p.rope_h = off; off += round_up((size_t)d.H * n2 * sizeof(float2), 256);
  p.rope_w = off; off += round_up((size_t)d.W * n2 * sizeof(float2), 256);
  p.rope_nz = off; off += round_up(n2 * sizeof(float), 256);
  p.tcode = off;  off += round_up((size_t)d.T * d.C * sizeof(float), 256);
  // channel gates: the x_proj and B_X kernels side by side as one (C, 2C) matrix
  const bool ch = d.gate_type == CSSM_GATE_CHANNEL;
  p.gw = off;     off += ch ? round_up((size_t)d.C * 2 * d.C * sizeof(float), 256) : 0;
  p.gb = off;     off += ch ? round_up((size_t)2 * d.C * sizeof(float), 256) : 0;
  p.total = off;
  return p;
}

struct AddWs { size_t planar, ctx_part, maps, dchan, cg, total; };
static AddWs additive_ws_layout(const cssm_additive_desc& d) {
  AddWs l;
  const size_t BT = (size_t)d.B * d.T, HW = (size_t)d.H * d.W, NB = (size_t)d.H * (d.W / 2 + 1);
  size_t off = 0;
  // (BT, 2C, H, W): the spectral kernels address the state planes with a stride of 2C planes
  // per frame; the upper C planes of a frame are not touched here
  l.planar = off;   off += round_up(BT * 2 * d.C * HW * sizeof(float), 256);
  l.ctx_part = off; off += round_up(BT * d.H * d.C * sizeof(float), 256);
  l.maps = off;     off += round_up(BT * NB * sizeof(float4), 256);
  const bool ch = d.gate_type == CSSM_GATE_CHANNEL;
  l.dchan = off;    off += ch ? round_up(BT * d.C * sizeof(float), 256) : 0;
  l.cg = off;       off += ch ? round_up(BT * d.C * HW * sizeof(float), 256) : 0;   // C_gate planes
  l.total = off;
  return l;
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_additive_plan_bytes(const cssm_additive_desc* d) {
  return additive_validate(d) == CSSM_OK ? additive_plan_layout(*d).total : 0;
}

size_t cssm_additive_workspace_bytes(const cssm_additive_desc* d) {
  return additive_validate(d) == CSSM_OK ? additive_ws_layout(*d).total : 0;
}

int cssm_additive_plan_init(const cssm_additive_desc* d, const cssm_additive_weights* w, void* plan,
                            size_t plan_bytes, void* stream) {
  int s = additive_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->kernel || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  const AddPlan p = additive_plan_layout(*d);
  if (plan_bytes < p.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = (char*)plan;
  // the log-space scan floors the magnitude of d_X * K_hat at 1e-7; here the floor acts on K_hat
  // before the gate (d_X lies in [0.1, 0.99]), a difference of at most 1e-7 in the transition
  s = launch_khat(w->kernel, (cf*)(base + p.khat), d->C, d->kernel_size, d->H, d->W,
                  d->spectral_rho, 1, d->goom_floor, spectral_path(d->H, d->W), st);
  if (s != CSSM_OK) return s;
  s = launch_rope_tables((float2*)(base + p.rope_t), (float2*)(base + p.rope_h),
                         (float2*)(base + p.rope_w), (float*)(base + p.rope_nz), d->T, d->H, d->W,
                         d->C, d->rope_mode, d->rope_base, st);
  if (s != CSSM_OK) return s;
  if (d->gate_type == CSSM_GATE_CHANNEL) {
    // [x_proj | B_X] -> one (C, 2C) matrix; gate_kernel[1] is the (1,1,C,C) conv kernel of B_X
    if (!w->x_proj_kernel || !w->x_proj_bias || !w->gate_kernel[1] || !w->gate_bias[1]) return CSSM_ERR_NULL;
    const size_t cb = (size_t)d->C * sizeof(float);
    const float* ks[2] = {w->x_proj_kernel, w->gate_kernel[1]};
    const float* bs[2] = {w->x_proj_bias, w->gate_bias[1]};
    for (int i = 0; i < 2; ++i) {
      cudaError_t e = cudaMemcpy2DAsync(base + p.gw + i * cb, 2 * cb, ks[i], cb, cb, (size_t)d->C,
                                        cudaMemcpyDeviceToDevice, st);
      if (e == cudaSuccess) e = cudaMemcpyAsync(base + p.gb + i * cb, bs[i], cb, cudaMemcpyDeviceToDevice, st);
      if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    }
  }
  return launch_tcode((float*)(base + p.tcode), d->T, d->C, d->rope_base, st);
}

int cssm_additive_forward(const cssm_additive_desc* d, const cssm_additive_weights* w,
                          const void* plan, const float* x, float* y, void* workspace,
                          size_t workspace_bytes, void* stream) {
  int s = additive_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan || !x || !y || !workspace) return CSSM_ERR_NULL;
  if (!w->x_proj_kernel || !w->x_proj_bias || !w->output_proj_kernel || !w->output_proj_bias)
    return CSSM_ERR_NULL;
  const bool chan = d->gate_type == CSSM_GATE_CHANNEL;
  const int nptr = d->gate_type == CSSM_GATE_FACTORED ? 6 : 3;
  for (int i = 0; i < nptr; ++i)
    if (!w->gate_kernel[i] || !w->gate_bias[i]) return CSSM_ERR_NULL;
  if (!aligned16(x) || !aligned16(y) || !aligned16(plan) || !aligned16(workspace))
    return CSSM_ERR_ALIGN;
  const AddWs l = additive_ws_layout(*d);
  if (workspace_bytes < l.total) return CSSM_ERR_WORKSPACE;
  const AddPlan p = additive_plan_layout(*d);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  const char* pl = (const char*)plan;
  const int BT = d->B * d->T, HW = d->H * d->W, C = d->C;
  const bool rope = d->rope_mode != CSSM_ROPE_NONE;
  const float2* rt = rope ? (const float2*)(pl + p.rope_t) : nullptr;
  const float2* rh = rope ? (const float2*)(pl + p.rope_h) : nullptr;
  const float2* rw = rope ? (const float2*)(pl + p.rope_w) : nullptr;
  const float* rnz = rope ? (const float*)(pl + p.rope_nz) : nullptr;
  float* planar = (float*)(ws + l.planar);

  // 1. context row sums of the rotated input
  GdnDwArgs dw;
  memset(&dw, 0, sizeof(dw));
  dw.x = x; dw.out = nullptr; dw.ksz = 1;
  dw.BT = BT; dw.T = d->T; dw.H = d->H; dw.W = d->W; dw.C = C;
  dw.rope_t = rt; dw.rope_h = rh; dw.rope_w = rw;
  dw.ctx_part = (float*)(ws + l.ctx_part);
  if ((s = launch_rope_dwconv_cl(dw, st)) != CSSM_OK) return s;

  // 2. x_proj of the rotated input -> the lower C planes of every frame (channel gates: the B_X
  //    map sigmoid(Conv1x1(x)) comes out of the same GEMM into the upper C planes)
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = BT * HW; g.N = chan ? 2 * C : C; g.K = C; g.HW = HW;
  g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
  g.Wk = chan ? (const float*)(pl + p.gw) : w->x_proj_kernel;
  g.bias = chan ? (const float*)(pl + p.gb) : w->x_proj_bias;
  g.out = planar; g.o_planes = 2 * C; g.o_plane0 = 0;
  g.T = d->T; g.H = d->H; g.W = d->W;
  if (chan) { g.out_act = 2; g.act_n0 = C; }
  if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;

  // 3. gate maps
  if (chan) {
    if (((size_t)C * HW) % 4 != 0) return CSSM_ERR_UNSUPPORTED;
    // x_proj *= B_X in the spatial domain
    const size_t per_frame4 = (size_t)C * HW / 4, total4 = per_frame4 * BT;
    additive_in_gate_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, st>>>(planar, per_frame4, total4);
    if ((s = check_launch()) != CSSM_OK) return s;
    AddChanArgs ca;
    memset(&ca, 0, sizeof(ca));
    ca.ctx_part = dw.ctx_part; ca.tcode = (const float*)(pl + p.tcode);
    ca.BT = BT; ca.T = d->T; ca.C = C; ca.H = d->H; ca.W = d->W; ca.goom_floor = d->goom_floor;
    ca.dk = w->gate_kernel[0]; ca.db = w->gate_bias[0];
    ca.dchan = (float*)(ws + l.dchan); ca.maps = (float4*)(ws + l.maps);
    additive_chan_gates_kernel<<<BT, 128, (size_t)C * sizeof(float), st>>>(ca);
    if ((s = check_launch()) != CSSM_OK) return s;
    // C_gate planes sigmoid(Conv1x1(rotated x))
    memset(&g, 0, sizeof(g));
    g.M = BT * HW; g.N = C; g.K = C; g.HW = HW;
    g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
    g.Wk = w->gate_kernel[2]; g.bias = w->gate_bias[2];
    g.out = (float*)(ws + l.cg); g.o_planes = C; g.o_plane0 = 0;
    g.T = d->T; g.H = d->H; g.W = d->W;
    g.out_act = 2; g.act_n0 = 0;
    if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;
  } else {
    AddGateArgs ga;
    memset(&ga, 0, sizeof(ga));
    ga.ctx_part = dw.ctx_part; ga.tcode = (const float*)(pl + p.tcode);
    ga.BT = BT; ga.T = d->T; ga.C = C; ga.H = d->H; ga.W = d->W;
    ga.gate_type = d->gate_type; ga.path = spectral_path(d->H, d->W); ga.goom_floor = d->goom_floor;
    for (int i = 0; i < nptr; ++i) { ga.gk[i] = w->gate_kernel[i]; ga.gb[i] = w->gate_bias[i]; }
    ga.maps = (float4*)(ws + l.maps);
    if ((s = launch_additive_gates(ga, st)) != CSSM_OK) return s;
  }

  // 4. fused rfft2 -> recurrence -> output gate -> irfft2, in place on the state planes
  s = launch_spectral(d->B, d->T, d->H, d->W, C, (const cf*)(pl + p.khat),
                      (const float*)(ws + l.maps), planar, 0, chan ? 3 : 2, st,
                      chan ? (const float*)(ws + l.dchan) : nullptr);
  if (s != CSSM_OK) return s;

  // 5. output_proj (channel gates: of the planes times C_gate) -> channels-last y
  memset(&g, 0, sizeof(g));
  g.M = BT * HW; g.N = C; g.K = C; g.HW = HW;
  g.A = planar; g.a_planes = 2 * C; g.a_plane0 = 0;
  if (chan) { g.gate = (const float*)(ws + l.cg); g.g_planes = C; g.g_plane0 = 0; }
  g.Wk = w->output_proj_kernel; g.bias = w->output_proj_bias;
  g.out = y;
  g.T = d->T; g.H = d->H; g.W = d->W;
  return launch_gemm<true, false>(g, st);
}

}  // extern "C"
