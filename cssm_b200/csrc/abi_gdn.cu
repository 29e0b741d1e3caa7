// extern "C" entry points of the GDN (GatedDeltaNetCSSM) block.
#include <string.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"

namespace cssm {

static SpectralPath gdn_path(const cssm_gdn_desc& d) {
  const SpectralPath p = spectral_path(d.H, d.W);
  return (p != PATH_GENERIC && d.delta_key_dim == 4) ? p : PATH_GENERIC;
}

struct GdnPlan { size_t what, rope_t, rope_h, rope_w, rope_nz, tcode, gw, gb, total; };
static GdnPlan gdn_plan_layout(const cssm_gdn_desc& d) {
  GdnPlan p;
  const size_t Wf = d.W / 2 + 1, n2 = d.C / 2, nh = d.C / d.delta_key_dim;
  size_t off = 0;
  p.what = off;   off += round_up(nh * d.H * Wf * sizeof(cf), 256);
  p.rope_t = off; off += round_up((size_t)d.T * n2 * sizeof(float2), 256);
  p.rope_h = off; off += round_up((size_t)d.H * n2 * sizeof(float2), 256);
  p.rope_w = off; off += round_up((size_t)d.W * n2 * sizeof(float2), 256);
  p.rope_nz = off; off += round_up(n2 * sizeof(float), 256);
  p.tcode = off;  off += round_up((size_t)d.T * d.C * sizeof(float), 256);
  // channel gates: the B_k, B_v 1x1-conv kernels packed side by side as one (C, 2C) matrix
  const bool chsp = d.gate_type == CSSM_GATE_CHANNEL && d.use_input_gates;
  p.gw = off;     off += chsp ? round_up((size_t)d.C * 2 * d.C * sizeof(float), 256) : 0;
  p.gb = off;     off += chsp ? round_up((size_t)2 * d.C * sizeof(float), 256) : 0;
  p.total = off;
  return p;
}

// k, v planes times their spatial gate planes: for every frame the 2C planes C..3C of the
// (frames, 3C, HW) q/k/v buffer are multiplied by the 2C planes of the (frames, 2C, HW) gate buffer
__global__ void __launch_bounds__(256) gdn_kv_gate_kernel(float* __restrict__ qkv, const float* __restrict__ gsp,
                                                          size_t per_frame4, size_t total4) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total4) return;
  const size_t fr = i / per_frame4, r = i - fr * per_frame4;
  float4* d = reinterpret_cast<float4*>(qkv) + fr * (per_frame4 + per_frame4 / 2) + per_frame4 / 2 + r;
  const float4 gv = __ldg(reinterpret_cast<const float4*>(gsp) + i);
  float4 v = *d;
  v.x *= gv.x; v.y *= gv.y; v.z *= gv.z; v.w *= gv.w;
  *d = v;
}

struct GdnWs { size_t xdw, qkv, gate, ctx_part, ab, bkv, gsp, state, total; };
static GdnWs gdn_ws_layout(const cssm_gdn_desc& d) {
  GdnWs l;
  const size_t BT = (size_t)d.B * d.T, HW = (size_t)d.H * d.W, NB = (size_t)d.H * (d.W / 2 + 1);
  const size_t nh = d.C / d.delta_key_dim, dk = d.delta_key_dim;
  size_t off = 0;
  l.xdw = off;      off += d.qkv_conv_size > 1 ? round_up(BT * HW * d.C * sizeof(float), 256) : 0;
  l.qkv = off;      off += round_up(BT * 3 * d.C * HW * sizeof(float), 256);
  l.gate = off;     off += round_up(BT * d.C * HW * sizeof(float), 256);
  l.ctx_part = off; off += round_up(BT * d.H * d.C * sizeof(float), 256);
  // channel gates: one {alpha, beta} map per (frame, head); the spatial input gates are planes
  const bool chan = d.gate_type == CSSM_GATE_CHANNEL;
  l.ab = off;       off += round_up(BT * (chan ? nh : 1) * NB * sizeof(float2), 256);
  l.bkv = off;      off += round_up(BT * HW * sizeof(float2), 256);
  l.gsp = off;      off += (chan && d.use_input_gates) ? round_up(BT * 2 * d.C * HW * sizeof(float), 256) : 0;
  l.state = off;    off += round_up((size_t)d.B * nh * dk * dk * NB * sizeof(cf), 256);
  l.total = off;
  return l;
}

static int gdn_validate(const cssm_gdn_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->kernel_size <= 0 ||
      d->delta_key_dim <= 0)
    return CSSM_ERR_DIMS;
  if (d->C % d->delta_key_dim != 0) return CSSM_ERR_DIMS;          // cssm.py:4690
  if (d->delta_key_dim > 4 || d->C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (d->rope_mode < CSSM_ROPE_NONE || d->rope_mode > CSSM_ROPE_MROPE) return CSSM_ERR_UNSUPPORTED;
  if (d->gate_type < CSSM_GATE_DENSE || d->gate_type > CSSM_GATE_SCALAR) return CSSM_ERR_UNSUPPORTED;
  if (d->short_conv_size < 0 || d->short_conv_size > 8) return CSSM_ERR_UNSUPPORTED;
  if (d->output_norm != 0 && d->output_norm != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->output_gate_act != 0 && d->output_gate_act != 1) return CSSM_ERR_UNSUPPORTED;
  if (d->qkv_conv_size < 1 || d->qkv_conv_size > 7 || d->qkv_conv_size % 2 == 0)
    return CSSM_ERR_UNSUPPORTED;
  const bool crop_h = d->kernel_size > d->H, crop_w = d->kernel_size > d->W;
  if (crop_h != crop_w) return CSSM_ERR_UNSUPPORTED;
  if (gdn_path(*d) == PATH_GENERIC &&
      gdn_generic_smem_bytes(d->H, d->W, d->delta_key_dim) > 220 * 1024)
    return CSSM_ERR_UNSUPPORTED;
  if ((size_t)d->qkv_conv_size * d->W * d->C * sizeof(float) > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  const size_t nhist = d->short_conv_size > 0 ? d->short_conv_size - 1 : 0;
  if ((1 + nhist) * d->H * d->W * sizeof(float) > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

// Stage events of the call in progress on this thread (cssm_gdn_forward_timed sets it for the
// duration of its own call only): events[i] is recorded on the stream before stage i
// (i = 0..6) and events[7] after the last stage.
static thread_local cudaEvent_t* g_stage_events = nullptr;
static inline void mark(int i, cudaStream_t st) {
  if (g_stage_events != nullptr && g_stage_events[i] != nullptr) cudaEventRecord(g_stage_events[i], st);
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_gdn_plan_bytes(const cssm_gdn_desc* d) {
  if (gdn_validate(d) != CSSM_OK) return 0;
  return gdn_plan_layout(*d).total;
}

size_t cssm_gdn_workspace_bytes(const cssm_gdn_desc* d) {
  if (gdn_validate(d) != CSSM_OK) return 0;
  return gdn_ws_layout(*d).total;
}

int cssm_gdn_plan_init(const cssm_gdn_desc* d, const cssm_gdn_weights* w, void* plan,
                       size_t plan_bytes, void* stream) {
  int s = gdn_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->kernel || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  const GdnPlan p = gdn_plan_layout(*d);
  if (plan_bytes < p.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = (char*)plan;
  // W_hat is NOT floored: in the reference the 1e-7 floor acts on the elements of M_t and
  // Delta_t (cssm.py:4947-4948), which this library never materialises.
  s = launch_khat(w->kernel, (cf*)(base + p.what), d->C / d->delta_key_dim, d->kernel_size, d->H,
                  d->W, d->spectral_rho, d->no_spectral_clamp ? 0 : 1, 0, gdn_path(*d), st);
  if (s != CSSM_OK) return s;
  s = launch_rope_tables((float2*)(base + p.rope_t), (float2*)(base + p.rope_h),
                         (float2*)(base + p.rope_w), (float*)(base + p.rope_nz), d->T, d->H, d->W,
                         d->C, d->rope_mode, d->rope_base, st);
  if (s != CSSM_OK) return s;
  if (d->gate_type == CSSM_GATE_CHANNEL && d->use_input_gates) {
    // gate_kernel[2], [3] = B_k, B_v 1x1-conv kernels (1,1,C,C) -> one (C, 2C) matrix
    const size_t cb = (size_t)d->C * sizeof(float);
    for (int i = 0; i < 2; ++i) {
      if (!w->gate_kernel[2 + i] || !w->gate_bias[2 + i]) return CSSM_ERR_NULL;
      cudaError_t e = cudaMemcpy2DAsync(base + p.gw + i * cb, 2 * cb, w->gate_kernel[2 + i], cb, cb,
                                        (size_t)d->C, cudaMemcpyDeviceToDevice, st);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(base + p.gb + i * cb, w->gate_bias[2 + i], cb, cudaMemcpyDeviceToDevice, st);
      if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    }
  }
  return launch_tcode((float*)(base + p.tcode), d->T, d->C, d->rope_base, st);
}

int cssm_gdn_forward(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                     const float* x, float* y, void* workspace, size_t workspace_bytes,
                     void* stream) {
  return gdn_forward_internal(d, w, plan, x, y, workspace, workspace_bytes, stream, 0, 0);
}

int cssm_gdn_forward_last(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                          const float* x, float* y_last, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return gdn_forward_internal(d, w, plan, x, y_last, workspace, workspace_bytes, stream, 1, 0);
}

int cssm_gdn_forward_static_image(const cssm_gdn_desc* d, const cssm_gdn_weights* w,
                                  const void* plan, const float* x, float* y, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  return gdn_forward_internal(d, w, plan, x, y, workspace, workspace_bytes, stream, 0, 2);
}

int cssm_gdn_forward_timed(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                           const float* x, float* y, void* workspace, size_t workspace_bytes,
                           void* stream, void** stage_events) {
  g_stage_events = reinterpret_cast<cudaEvent_t*>(stage_events);
  const int s = gdn_forward_internal(d, w, plan, x, y, workspace, workspace_bytes, stream, 0, 0);
  g_stage_events = nullptr;
  return s;
}

}  // extern "C"

// last_only != 0: y is (B,H,W,C), the last frame of the block output.  The gate projection, the
// readout, the inverse transforms, RMSNorm and the output projection then run for the last
// frame of every batch element only; q/k/v, the gate maps and the state recurrence cover all T.
// x_bcast != 0: x is (B,H,W,C), one frame per batch element standing for all T frames.
// x_bcast == 2: static-image fast path (cssm.py:4353-4683): x and y are (B,H,W,C), d->T is the
// number of gate steps; q, k, v and gate_val are computed once per image, the gates for all T.
int cssm::gdn_forward_internal(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                               const float* x, float* y, void* workspace, size_t workspace_bytes,
                               void* stream, int last_only, int x_bcast) {
  const int static_image = x_bcast == 2 ? 1 : 0;
  if (static_image) {
    x_bcast = 0;
    if (last_only) return CSSM_ERR_UNSUPPORTED;
    // preconditions asserted by the reference (cssm.py:4354-4370)
    if (d && (d->short_conv_size != 0 || d->use_input_gates != 0 || d->rope_mode != CSSM_ROPE_NONE))
      return CSSM_ERR_UNSUPPORTED;
    if (d && d->gate_type >= CSSM_GATE_CHANNEL) return CSSM_ERR_UNSUPPORTED;   // dense and factored maps only
  }
  int s = gdn_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan || !x || !y || !workspace) return CSSM_ERR_NULL;
  if (!w->kernel || !w->qkv_proj_kernel || !w->qkv_proj_bias || !w->gate_proj_kernel ||
      !w->gate_proj_bias || !w->output_proj_kernel || !w->output_proj_bias)
    return CSSM_ERR_NULL;
  if (d->qkv_conv_size > 1 && (!w->qkv_dw_kernel || !w->qkv_dw_bias)) return CSSM_ERR_NULL;
  if (d->output_norm == 1 && !w->rms_scale) return CSSM_ERR_NULL;
  if (d->short_conv_size > 0)
    for (int i = 0; i < 3; ++i)
      if (!w->conv_t_kernel[i] || !w->conv_t_bias[i]) return CSSM_ERR_NULL;
  const bool chan = d->gate_type == CSSM_GATE_CHANNEL;
  const int ngate = d->use_input_gates ? 4 : 2;
  const int nptr = d->gate_type == CSSM_GATE_FACTORED ? 2 * ngate : ngate;
  for (int i = 0; i < nptr; ++i)
    if (!w->gate_kernel[i] || !w->gate_bias[i]) return CSSM_ERR_NULL;
  if (!aligned16(x) || !aligned16(y) || !aligned16(plan) || !aligned16(workspace))
    return CSSM_ERR_ALIGN;
  const GdnWs l = gdn_ws_layout(*d);
  if (workspace_bytes < l.total) return CSSM_ERR_WORKSPACE;
  const GdnPlan p = gdn_plan_layout(*d);
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  const char* pl = (const char*)plan;
  const int Tdata = static_image ? 1 : d->T;            // frames of x per batch element
  const int BT = d->B * Tdata, HW = d->H * d->W, C = d->C;
  const bool rope = d->rope_mode != CSSM_ROPE_NONE;
  const float2* rt = rope ? (const float2*)(pl + p.rope_t) : nullptr;
  const float2* rh = rope ? (const float2*)(pl + p.rope_h) : nullptr;
  const float2* rw = rope ? (const float2*)(pl + p.rope_w) : nullptr;
  const float* rnz = rope ? (const float*)(pl + p.rope_nz) : nullptr;
  float* xdw = (float*)(ws + l.xdw);
  float* qkv = (float*)(ws + l.qkv);
  float* gate = (float*)(ws + l.gate);

  // 1. RoPE + depthwise conv (channels-last) and the context row sums of the rotated input
  mark(0, st);
  GdnDwArgs dw;
  memset(&dw, 0, sizeof(dw));
  dw.x = x; dw.out = d->qkv_conv_size > 1 ? xdw : nullptr;
  dw.wk = w->qkv_dw_kernel; dw.bias = w->qkv_dw_bias; dw.ksz = d->qkv_conv_size;
  dw.BT = BT; dw.T = Tdata; dw.H = d->H; dw.W = d->W; dw.C = C; dw.x_bcast = x_bcast;
  dw.rope_t = rt; dw.rope_h = rh; dw.rope_w = rw;
  dw.ctx_part = (float*)(ws + l.ctx_part);
  if ((s = launch_rope_dwconv_cl(dw, st)) != CSSM_OK) return s;

  // 2. qkv projection -> planar (BT, 3C, H, W)
  mark(1, st);
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = BT * HW; g.N = 3 * C; g.K = C; g.HW = HW;
  g.Wk = w->qkv_proj_kernel; g.bias = w->qkv_proj_bias;
  g.out = qkv; g.o_planes = 3 * C; g.o_plane0 = 0;
  g.T = Tdata; g.H = d->H; g.W = d->W;
  if (d->qkv_conv_size > 1) { g.A = xdw; }
  else {
    g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
    if (x_bcast) { g.a_fdiv = d->T; g.a_fmul = 1; g.a_fadd = 0; }
  }
  if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;

  // 3. output gate projection of the rotated input -> planar, through SiLU / sigmoid
  //    (last_only: rows of frame T-1 of every batch element -> planes (B, C, H, W))
  mark(2, st);
  const int Mout = last_only ? d->B * HW : BT * HW;
  memset(&g, 0, sizeof(g));
  g.M = Mout; g.N = C; g.K = C; g.HW = HW;
  if (last_only) {
    g.rope_tlast = 1;
    if (!x_bcast) { g.a_fmul = d->T; g.a_fadd = d->T - 1; }     // else frame b is the source
  } else if (x_bcast) {
    g.a_fdiv = d->T; g.a_fmul = 1; g.a_fadd = 0;
  }
  g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
  g.Wk = w->gate_proj_kernel; g.bias = w->gate_proj_bias;
  g.out = gate; g.o_planes = C; g.o_plane0 = 0;
  g.T = Tdata; g.H = d->H; g.W = d->W;
  g.out_act = d->output_gate_act == 0 ? 1 : 2;
  if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;

  // 4. gate maps
  mark(3, st);
  GdnGateArgs ga;
  memset(&ga, 0, sizeof(ga));
  ga.ctx_part = dw.ctx_part; ga.tcode = (const float*)(pl + p.tcode);
  ga.BT = d->B * d->T; ga.T = d->T; ga.C = C; ga.H = d->H; ga.W = d->W;
  ga.ctx_per_clip = static_image;
  ga.gate_type = d->gate_type; ga.use_input_gates = d->use_input_gates; ga.path = gdn_path(*d);
  ga.nh = C / d->delta_key_dim;
  for (int i = 0; i < nptr; ++i) { ga.gk[i] = w->gate_kernel[i]; ga.gb[i] = w->gate_bias[i]; }
  ga.ab = (float2*)(ws + l.ab); ga.bkv = (float2*)(ws + l.bkv);
  if ((s = launch_gdn_gates(ga, st)) != CSSM_OK) return s;

  // 5. causal temporal conv + SiLU on q, k, v planes, input gates on k and v
  mark(4, st);
  bool tconv_done = false;
  // one elementwise launch over q, k, v where it measured faster than three per-plane launches
  // (64x64 planes: 1.70 -> 1.36 ms on B=128, T=8; at 32x32 the per-plane kernel is ahead)
  if (d->short_conv_size >= 2 && d->short_conv_size <= 4 && HW % 4 == 0 && HW != 1024) {
    QkvTconvArgs ta;
    memset(&ta, 0, sizeof(ta));
    ta.buf = qkv; ta.B = d->B; ta.T = Tdata; ta.C = C; ta.HW = HW; ta.kt = d->short_conv_size;
    for (int i = 0; i < 3; ++i) { ta.wt[i] = w->conv_t_kernel[i]; ta.bt[i] = w->conv_t_bias[i]; }
    ta.bkv = (d->use_input_gates && !chan) ? (const float2*)(ws + l.bkv) : nullptr;
    s = launch_qkv_temporal_conv(ta, st);
    if (s == CSSM_OK) tconv_done = true;
    else if (s != CSSM_ERR_UNSUPPORTED) return s;
  }
  for (int i = 0; i < 3 && !tconv_done; ++i) {
    const bool has_post = d->use_input_gates && !chan && i > 0;
    if (d->short_conv_size == 0 && !has_post) continue;
    StencilArgs sa;
    memset(&sa, 0, sizeof(sa));
    sa.buf = qkv; sa.planes_per_frame = 3 * C; sa.plane0 = i * C;
    sa.B = d->B; sa.T = Tdata; sa.C = C; sa.H = d->H; sa.W = d->W;
    sa.ksp = 0; sa.kt = d->short_conv_size;
    sa.wt = w->conv_t_kernel[i]; sa.bt = w->conv_t_bias[i];
    sa.act = d->short_conv_size > 0 ? 1 : 0;
    if (has_post) { sa.post = (const float*)(ws + l.bkv); sa.post_stride = 2; sa.post_off = i - 1; }
    if ((s = launch_plane_stencil(sa, st)) != CSSM_OK) return s;
  }

  if (chan && d->use_input_gates) {
    // spatial gates sigmoid(Conv1x1(rotated x)) -> planes (BT, 2C, H, W): B_k, B_v; k *= B_k, v *= B_v
    float* gsp = (float*)(ws + l.gsp);
    memset(&g, 0, sizeof(g));
    g.M = BT * HW; g.N = 2 * C; g.K = C; g.HW = HW;
    g.A = x; g.rope_t = rt; g.rope_h = rh; g.rope_w = rw; g.rope_nz = rnz;
    if (x_bcast) { g.a_fdiv = d->T; g.a_fmul = 1; g.a_fadd = 0; }
    g.Wk = (const float*)(pl + p.gw); g.bias = (const float*)(pl + p.gb);      // packed by plan_init
    g.out = gsp; g.o_planes = 2 * C; g.o_plane0 = 0;
    g.T = Tdata; g.H = d->H; g.W = d->W;
    g.out_act = 2; g.act_n0 = 0;
    if ((s = launch_gemm<false, true>(g, st)) != CSSM_OK) return s;
    if (((size_t)C * HW) % 8 != 0) return CSSM_ERR_UNSUPPORTED;
    const size_t per_frame4 = (size_t)2 * C * HW / 4, total4 = per_frame4 * BT;
    gdn_kv_gate_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, st>>>(qkv, gsp, per_frame4, total4);
    if ((s = check_launch()) != CSSM_OK) return s;
  }

  // 6. fused spectral recurrence; the output planes overwrite the v planes
  mark(5, st);
  GdnSpectralArgs sp;
  memset(&sp, 0, sizeof(sp));
  sp.qkv = qkv; sp.what = (const cf*)(pl + p.what); sp.ab = ga.ab; sp.state = (cf*)(ws + l.state);
  sp.ab_heads = chan ? C / d->delta_key_dim : 1;
  sp.B = d->B; sp.T = d->T; sp.C = C; sp.H = d->H; sp.W = d->W; sp.dk = d->delta_key_dim;
  sp.use_l2 = d->use_spectral_l2_norm;
  sp.last_only = last_only;
  sp.static_image = static_image;
  if ((s = launch_gdn_spectral(sp, st)) != CSSM_OK) return s;

  // 7. RMSNorm over channels, output gate, output projection -> channels-last y
  mark(6, st);
  memset(&g, 0, sizeof(g));
  g.M = Mout; g.N = C; g.K = C; g.HW = HW;
  g.A = qkv; g.a_planes = 3 * C; g.a_plane0 = 2 * C;
  if (last_only) { g.a_fmul = d->T; g.a_fadd = d->T - 1; g.g_compact = 1; }
  g.rms_scale = d->output_norm == 1 ? w->rms_scale : nullptr;
  g.gate = gate; g.g_planes = C; g.g_plane0 = 0;
  g.Wk = w->output_proj_kernel; g.bias = w->output_proj_bias;
  g.out = y;
  g.T = Tdata; g.H = d->H; g.W = d->W;
  s = launch_gemm<true, false>(g, st);
  mark(7, st);
  return s;
}
