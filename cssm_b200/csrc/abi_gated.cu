// extern "C" entry points of the gated (GatedCSSM) block and the shared error plumbing.
#include <string.h>
#include <stdio.h>
#include <cuda_bf16.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"

namespace cssm {

static thread_local char g_cuda_err[256] = "";

void set_cuda_error(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
}

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

SpectralPath spectral_path(int H, int W) {
  if (H == 64 && W == 64) return PATH_R64;
  if (H == 32 && W == 32) return PATH_R32;
  return PATH_GENERIC;
}

GatedPlan gated_plan_layout(const cssm_gated_desc& d) {
  GatedPlan p;
  const size_t Wf = d.W / 2 + 1, n2 = d.C / 2;
  size_t off = 0;
  p.khat = off;   off += round_up((size_t)d.C * d.H * Wf * sizeof(cf), 256);
  p.rope_t = off; off += round_up((size_t)d.T * n2 * sizeof(float2), 256);
  p.rope_h = off; off += round_up((size_t)d.H * n2 * sizeof(float2), 256);
  p.rope_w = off; off += round_up((size_t)d.W * n2 * sizeof(float2), 256);
  p.rope_nz = off; off += round_up(n2 * sizeof(float), 256);
  p.total = off;
  return p;
}



static int validate(const cssm_gated_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->kernel_size <= 0)
    return CSSM_ERR_DIMS;
  if (d->C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (d->rope_mode < CSSM_ROPE_NONE || d->rope_mode > CSSM_ROPE_MROPE) return CSSM_ERR_UNSUPPORTED;
  if (d->gate_type != CSSM_GATE_DENSE && d->gate_type != CSSM_GATE_FACTORED)
    return CSSM_ERR_UNSUPPORTED;
  if (d->gate_activation < 0 || d->gate_activation > CSSM_ACT_EXP_CLIP) return CSSM_ERR_UNSUPPORTED;
  if (d->short_conv_size < 0 || d->short_conv_size > 8) return CSSM_ERR_UNSUPPORTED;
  if (d->short_conv_spatial_size < 0 || d->short_conv_spatial_size > 7 ||
      (d->short_conv_spatial_size > 0 && d->short_conv_spatial_size % 2 == 0))
    return CSSM_ERR_UNSUPPORTED;
  const bool crop_h = d->kernel_size > d->H, crop_w = d->kernel_size > d->W;
  if (crop_h != crop_w) return CSSM_ERR_UNSUPPORTED;
  if (spectral_path(d->H, d->W) == PATH_GENERIC && generic_smem_bytes(d->H, d->W) > 200 * 1024)
    return CSSM_ERR_UNSUPPORTED;
  const size_t nh = d->short_conv_size > 0 ? d->short_conv_size - 1 : 0;
  if ((1 + nh) * d->H * d->W * sizeof(float) > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

static int validate_weights(const cssm_gated_desc* d, const cssm_gated_weights* w) {
  if (!w) return CSSM_ERR_NULL;
  if (!w->in_proj_kernel || !w->in_proj_bias || !w->kernel || !w->out_proj_kernel ||
      !w->out_proj_bias)
    return CSSM_ERR_NULL;
  if (d->short_conv_spatial_size > 0 && (!w->conv_sp_kernel || !w->conv_sp_bias)) return CSSM_ERR_NULL;
  if (d->short_conv_size > 0 && (!w->conv_t_kernel || !w->conv_t_bias)) return CSSM_ERR_NULL;
  const int ng = d->gate_type == CSSM_GATE_FACTORED ? 6 : 3;
  for (int i = 0; i < ng; ++i)
    if (!w->gate_kernel[i] || !w->gate_bias[i]) return CSSM_ERR_NULL;
  return CSSM_OK;
}

static void ws_layout(const cssm_gated_desc& d, cssm_gated_ws_layout* l) {
  const size_t BT = (size_t)d.B * d.T, HW = (size_t)d.H * d.W, NB = (size_t)d.H * (d.W / 2 + 1);
  size_t off = 0;
  l->xz_planar = off; off += round_up(BT * 2 * d.C * HW * sizeof(float), 256);
  l->ctx_sum = off;   off += round_up(BT * d.C * sizeof(float), 256);
  l->gate_maps = off; off += round_up(BT * NB * 4 * sizeof(float), 256);
  l->total = off;
}

}  // namespace cssm

using namespace cssm;

extern "C" {

const char* cssm_strerror(int s) {
  switch (s) {
    case CSSM_OK: return "ok";
    case CSSM_ERR_NULL: return "required pointer is NULL";
    case CSSM_ERR_DIMS: return "bad dimensions";
    case CSSM_ERR_UNSUPPORTED: return "unsupported field combination";
    case CSSM_ERR_ALIGN: return "pointer not 16-byte aligned";
    case CSSM_ERR_WORKSPACE: return "plan or workspace buffer too small";
    case CSSM_ERR_CUDA: return "CUDA error";
    case CSSM_ERR_SIZE_LIMIT: return "size beyond a fixed maximum";
    default: return "unknown status";
  }
}

const char* cssm_last_cuda_error(void) { return g_cuda_err; }
const char* cssm_version(void) { return "cssm_b200 0.1 sm_100a"; }

size_t cssm_gated_plan_bytes(const cssm_gated_desc* d) {
  if (validate(d) != CSSM_OK) return 0;
  return gated_plan_layout(*d).total;
}

int cssm_gated_workspace_layout(const cssm_gated_desc* d, cssm_gated_ws_layout* out) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!out) return CSSM_ERR_NULL;
  ws_layout(*d, out);
  return CSSM_OK;
}

size_t cssm_gated_workspace_bytes(const cssm_gated_desc* d) {
  if (validate(d) != CSSM_OK) return 0;
  cssm_gated_ws_layout l;
  ws_layout(*d, &l);
  return l.total;
}

int cssm_gated_plan_init(const cssm_gated_desc* d, const cssm_gated_weights* w, void* plan,
                         size_t plan_bytes, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->kernel || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  const GatedPlan p = gated_plan_layout(*d);
  if (plan_bytes < p.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = (char*)plan;
  s = launch_khat(w->kernel, (cf*)(base + p.khat), d->C, d->kernel_size, d->H, d->W,
                  d->spectral_rho, 1, 1, spectral_path(d->H, d->W), st);
  if (s != CSSM_OK) return s;
  return launch_rope_tables((float2*)(base + p.rope_t), (float2*)(base + p.rope_h),
                            (float2*)(base + p.rope_w), (float*)(base + p.rope_nz), d->T, d->H,
                            d->W, d->C, d->rope_mode, d->rope_base, st);
}

static int gated_in_proj_impl(const cssm_gated_desc* d, const cssm_gated_weights* w,
                              const void* plan, const float* x, float* xz, void* stream,
                              int x_bcast, int z_last_only = 0);

int cssm_gated_in_proj(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                       const float* x, float* xz, void* stream) {
  return gated_in_proj_impl(d, w, plan, x, xz, stream, 0);
}

// x_bcast != 0: x is (B,H,W,C), one frame per batch element that stands for all T frames
// z_last_only != 0: the silu(z) planes are only written for the last frame of every clip
static int gated_in_proj_impl(const cssm_gated_desc* d, const cssm_gated_weights* w,
                              const void* plan, const float* x, float* xz, void* stream,
                              int x_bcast, int z_last_only) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->in_proj_kernel || !w->in_proj_bias || !plan || !x || !xz) return CSSM_ERR_NULL;
  if (!aligned16(x) || !aligned16(xz) || !aligned16(plan)) return CSSM_ERR_ALIGN;
  const GatedPlan p = gated_plan_layout(*d);
  const char* base = (const char*)plan;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = d->B * d->T * d->H * d->W; g.N = 2 * d->C; g.K = d->C; g.HW = d->H * d->W;
  g.A = x; g.Wk = w->in_proj_kernel; g.bias = w->in_proj_bias;
  g.out = xz; g.o_planes = 2 * d->C; g.o_plane0 = 0;
  g.out_act = 1; g.act_n0 = d->C;          // the z planes are stored as silu(z)
  if (d->rope_mode != CSSM_ROPE_NONE) {
    g.rope_t = (const float2*)(base + p.rope_t);
    g.rope_h = (const float2*)(base + p.rope_h);
    g.rope_w = (const float2*)(base + p.rope_w);
    g.rope_nz = (const float*)(base + p.rope_nz);
  }
  g.T = d->T; g.H = d->H; g.W = d->W;
  if (x_bcast) { g.a_fdiv = d->T; g.a_fmul = 1; g.a_fadd = 0; }
  g.z_last_only = z_last_only;
  return launch_gemm<false, true>(g, (cudaStream_t)stream);
}

int cssm_gated_short_conv(const cssm_gated_desc* d, const cssm_gated_weights* w, float* xz,
                          float* ctx_sum, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !xz || !ctx_sum) return CSSM_ERR_NULL;
  if (d->short_conv_spatial_size > 0 && (!w->conv_sp_kernel || !w->conv_sp_bias)) return CSSM_ERR_NULL;
  if (d->short_conv_size > 0 && (!w->conv_t_kernel || !w->conv_t_bias)) return CSSM_ERR_NULL;
  StencilArgs a;
  memset(&a, 0, sizeof(a));
  a.buf = xz; a.planes_per_frame = 2 * d->C; a.plane0 = 0;
  a.B = d->B; a.T = d->T; a.C = d->C; a.H = d->H; a.W = d->W;
  a.wsp = w->conv_sp_kernel; a.bsp = w->conv_sp_bias; a.ksp = d->short_conv_spatial_size;
  a.wt = w->conv_t_kernel; a.bt = w->conv_t_bias; a.kt = d->short_conv_size;
  a.act = 1; a.post = nullptr; a.sums = ctx_sum;
  return launch_plane_stencil(a, (cudaStream_t)stream);
}

int cssm_gated_gates(const cssm_gated_desc* d, const cssm_gated_weights* w, const float* ctx_sum,
                     float* gate_maps, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !ctx_sum || !gate_maps) return CSSM_ERR_NULL;
  if (!aligned16(gate_maps)) return CSSM_ERR_ALIGN;
  const int ng = d->gate_type == CSSM_GATE_FACTORED ? 6 : 3;
  GatedGateArgs g;
  memset(&g, 0, sizeof(g));
  for (int i = 0; i < ng; ++i) {
    if (!w->gate_kernel[i] || !w->gate_bias[i]) return CSSM_ERR_NULL;
    g.gk[i] = w->gate_kernel[i]; g.gb[i] = w->gate_bias[i];
  }
  g.ctx_sum = ctx_sum; g.BT = d->B * d->T; g.C = d->C; g.H = d->H; g.W = d->W;
  g.gate_type = d->gate_type; g.act = d->gate_activation; g.path = spectral_path(d->H, d->W);
  g.maps = (float4*)gate_maps;
  return launch_gated_gates(g, (cudaStream_t)stream);
}

int cssm_gated_spectral(const cssm_gated_desc* d, const void* plan, const float* gate_maps,
                        float* xz, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!plan || !gate_maps || !xz) return CSSM_ERR_NULL;
  if (!aligned16(plan) || !aligned16(gate_maps) || !aligned16(xz)) return CSSM_ERR_ALIGN;
  const GatedPlan p = gated_plan_layout(*d);
  return launch_gated_spectral(*d, (const cf*)((const char*)plan + p.khat), gate_maps, xz, 0,
                               (cudaStream_t)stream);
}

int cssm_gated_out_proj(const cssm_gated_desc* d, const cssm_gated_weights* w, const float* xz,
                        float* y, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->out_proj_kernel || !w->out_proj_bias || !xz || !y) return CSSM_ERR_NULL;
  if (!aligned16(xz) || !aligned16(y)) return CSSM_ERR_ALIGN;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = d->B * d->T * d->H * d->W; g.N = d->C; g.K = d->C; g.HW = d->H * d->W;
  g.A = xz; g.a_planes = 2 * d->C; g.a_plane0 = 0;
  g.Wk = w->out_proj_kernel; g.bias = w->out_proj_bias;
  g.out = y;
  g.T = d->T; g.H = d->H; g.W = d->W;
  return launch_gemm<true, false>(g, (cudaStream_t)stream);
}

}  // extern "C"

namespace cssm {
int gated_forward_internal(const cssm_gated_desc* d, const cssm_gated_weights* w,
                           const void* plan, const float* x, float* y, void* workspace,
                           size_t workspace_bytes, void* stream, int last_only, int x_bcast) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  s = validate_weights(d, w);
  if (s != CSSM_OK) return s;
  if (!plan || !x || !y || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(workspace) || !aligned16(plan) || !aligned16(x) || !aligned16(y)) return CSSM_ERR_ALIGN;
  cssm_gated_ws_layout l;
  ws_layout(*d, &l);
  if (workspace_bytes < l.total) return CSSM_ERR_WORKSPACE;
  char* ws = (char*)workspace;
  float* xz = (float*)(ws + l.xz_planar);
  float* ctx = (float*)(ws + l.ctx_sum);
  float* gm = (float*)(ws + l.gate_maps);
  if ((s = gated_in_proj_impl(d, w, plan, x, xz, stream, x_bcast, last_only)) != CSSM_OK) return s;
  if ((s = cssm_gated_short_conv(d, w, xz, ctx, stream)) != CSSM_OK) return s;
  if ((s = cssm_gated_gates(d, w, ctx, gm, stream)) != CSSM_OK) return s;
  if (!last_only) {
    if ((s = cssm_gated_spectral(d, plan, gm, xz, stream)) != CSSM_OK) return s;
    return cssm_gated_out_proj(d, w, xz, y, stream);
  }
  const GatedPlan p = gated_plan_layout(*d);
  s = launch_gated_spectral(*d, (const cf*)((const char*)plan + p.khat), gm, xz, 1,
                            (cudaStream_t)stream);
  if (s != CSSM_OK) return s;
  // out_proj of the last frame of every batch element only
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = d->B * d->H * d->W; g.N = d->C; g.K = d->C; g.HW = d->H * d->W;
  g.A = xz; g.a_planes = 2 * d->C; g.a_plane0 = 0;
  g.a_fmul = d->T; g.a_fadd = d->T - 1;
  g.Wk = w->out_proj_kernel; g.bias = w->out_proj_bias;
  g.out = y;
  g.T = 1; g.H = d->H; g.W = d->W;
  return launch_gemm<true, false>(g, (cudaStream_t)stream);
}
}  // namespace cssm

extern "C" {

int cssm_gated_forward(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                       const float* x, float* y, void* workspace, size_t workspace_bytes,
                       void* stream) {
  return gated_forward_internal(d, w, plan, x, y, workspace, workspace_bytes, stream, 0, 0);
}

int cssm_gated_forward_last(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                            const float* x, float* y_last, void* workspace, size_t workspace_bytes,
                            void* stream) {
  return gated_forward_internal(d, w, plan, x, y_last, workspace, workspace_bytes, stream, 1, 0);
}

}  // extern "C"

// ------------------------------------------------------------ bf16 activations ----
namespace cssm {
// 8 elements per thread; n8 = number of 8-element groups, tail handled by the last threads
__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in,
                                                          float* __restrict__ out, size_t n) {
  const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const uint4 v = *reinterpret_cast<const uint4*>(in + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float4 a, b;
    float2 t;
    t = __bfloat1622float2(h[0]); a.x = t.x; a.y = t.y;
    t = __bfloat1622float2(h[1]); a.z = t.x; a.w = t.y;
    t = __bfloat1622float2(h[2]); b.x = t.x; b.y = t.y;
    t = __bfloat1622float2(h[3]); b.z = t.x; b.w = t.y;
    *reinterpret_cast<float4*>(out + i) = a;
    *reinterpret_cast<float4*>(out + i + 4) = b;
  } else {
    for (size_t j = i; j < n; ++j) out[j] = __bfloat162float(in[j]);
  }
}
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ in,
                                                          __nv_bfloat16* __restrict__ out, size_t n) {
  const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(in + i);
    const float4 b = *reinterpret_cast<const float4*>(in + i + 4);
    __nv_bfloat162 h[4];
    h[0] = __floats2bfloat162_rn(a.x, a.y); h[1] = __floats2bfloat162_rn(a.z, a.w);
    h[2] = __floats2bfloat162_rn(b.x, b.y); h[3] = __floats2bfloat162_rn(b.z, b.w);
    *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(h);
  } else {
    for (size_t j = i; j < n; ++j) out[j] = __float2bfloat16_rn(in[j]);
  }
}
}  // namespace cssm

extern "C" {

size_t cssm_gated_bf16_workspace_bytes(const cssm_gated_desc* d) {
  const size_t base = cssm_gated_workspace_bytes(d);
  if (base == 0) return 0;
  const size_t act = round_up((size_t)d->B * d->T * d->H * d->W * d->C * sizeof(float), 256);
  return base + 2 * act;
}

int cssm_gated_forward_bf16(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                            const void* x_bf16, void* y, int32_t y_is_bf16, void* workspace,
                            size_t workspace_bytes, void* stream) {
  void* y_bf16 = y;
  const size_t base = cssm_gated_workspace_bytes(d);
  if (base == 0) return validate(d) != CSSM_OK ? validate(d) : CSSM_ERR_DIMS;
  if (!x_bf16 || !y || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(x_bf16) || !aligned16(y) || !aligned16(workspace)) return CSSM_ERR_ALIGN;
  if (workspace_bytes < cssm_gated_bf16_workspace_bytes(d)) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = (size_t)d->B * d->T * d->H * d->W * d->C;
  const size_t act = round_up(n * sizeof(float), 256);
  char* ws = (char*)workspace;
  float* xf = (float*)(ws + base);
  float* yf = (float*)(ws + base + act);
  const unsigned grid = (unsigned)((n + 2047) / 2048);
  bf16_to_f32_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x_bf16, xf, n);
  int s = check_launch();
  if (s != CSSM_OK) return s;
  // float32 result (what Flax's promotion gives the reference) straight into y, or rounded to bf16
  s = gated_forward_internal(d, w, plan, xf, y_is_bf16 ? yf : (float*)y, workspace, base, stream, 0, 0);
  if (s != CSSM_OK || !y_is_bf16) return s;
  f32_to_bf16_kernel<<<grid, 256, 0, st>>>(yf, (__nv_bfloat16*)y_bf16, n);
  return check_launch();
}

}  // extern "C"

// ------------------------------------------------------------ host-buffer variant ----
namespace cssm {
struct HostChunkLayout { size_t x, y, ws, per_set, total; };
static HostChunkLayout host_layout(const cssm_gated_desc& d, int chunk_b) {
  cssm_gated_desc c = d;
  c.B = chunk_b;
  cssm_gated_ws_layout l;
  ws_layout(c, &l);
  HostChunkLayout h;
  const size_t act = round_up((size_t)chunk_b * d.T * d.H * d.W * d.C * sizeof(float), 256);
  h.x = 0; h.y = act; h.ws = 2 * act; h.per_set = 2 * act + l.total; h.total = 2 * h.per_set;
  return h;
}
}  // namespace cssm

extern "C" {

size_t cssm_gated_host_workspace_bytes(const cssm_gated_desc* d, int32_t chunk_b) {
  if (validate(d) != CSSM_OK || chunk_b <= 0) return 0;
  return host_layout(*d, chunk_b < d->B ? chunk_b : d->B).total;
}

int cssm_gated_forward_host(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                            const float* x_host, float* y_host, int32_t chunk_b, void* workspace,
                            size_t workspace_bytes, void* stream) {
  int s = validate(d);
  if (s != CSSM_OK) return s;
  s = validate_weights(d, w);
  if (s != CSSM_OK) return s;
  if (!plan || !x_host || !y_host || !workspace) return CSSM_ERR_NULL;
  if (chunk_b <= 0) return CSSM_ERR_DIMS;
  if (chunk_b > d->B) chunk_b = d->B;
  if (!aligned16(workspace)) return CSSM_ERR_ALIGN;
  const HostChunkLayout hl = host_layout(*d, chunk_b);
  if (workspace_bytes < hl.total) return CSSM_ERR_WORKSPACE;

  cudaStream_t user = (cudaStream_t)stream;
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_comp[2] = {nullptr, nullptr},
              ev_out[2] = {nullptr, nullptr}, ev_start = nullptr;
  int rc = CSSM_OK;
  cudaError_t e = cudaSuccess;
  auto fail = [&](cudaError_t err) { set_cuda_error(err); rc = CSSM_ERR_CUDA; };
#define CSSM_TRY(call) do { if (rc == CSSM_OK) { e = (call); if (e != cudaSuccess) fail(e); } } while (0)
  CSSM_TRY(cudaStreamCreateWithFlags(&s_in, cudaStreamNonBlocking));
  CSSM_TRY(cudaStreamCreateWithFlags(&s_out, cudaStreamNonBlocking));
  CSSM_TRY(cudaEventCreateWithFlags(&ev_start, cudaEventDisableTiming));
  for (int i = 0; i < 2; ++i) {
    CSSM_TRY(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
    CSSM_TRY(cudaEventCreateWithFlags(&ev_comp[i], cudaEventDisableTiming));
    CSSM_TRY(cudaEventCreateWithFlags(&ev_out[i], cudaEventDisableTiming));
  }
  // copies start only after work already queued on the caller's stream (e.g. plan_init)
  CSSM_TRY(cudaEventRecord(ev_start, user));
  CSSM_TRY(cudaStreamWaitEvent(s_in, ev_start, 0));

  const size_t per_b = (size_t)d->T * d->H * d->W * d->C;
  const int nchunk = (d->B + chunk_b - 1) / chunk_b;
  for (int i = 0; i < nchunk && rc == CSSM_OK; ++i) {
    const int set = i & 1;
    const int b0 = i * chunk_b;
    const int cb = (d->B - b0) < chunk_b ? (d->B - b0) : chunk_b;
    char* base = (char*)workspace + (size_t)set * hl.per_set;
    float* xd = (float*)(base + hl.x);
    float* yd = (float*)(base + hl.y);
    cssm_gated_desc c = *d;
    c.B = cb;
    cssm_gated_ws_layout l;
    ws_layout(c, &l);
    if (i >= 2) {
      CSSM_TRY(cudaStreamWaitEvent(s_in, ev_comp[set], 0));   // x buffer free again
      CSSM_TRY(cudaStreamWaitEvent(user, ev_out[set], 0));    // y buffer drained
    }
    CSSM_TRY(cudaMemcpyAsync(xd, x_host + (size_t)b0 * per_b, (size_t)cb * per_b * sizeof(float),
                             cudaMemcpyHostToDevice, s_in));
    CSSM_TRY(cudaEventRecord(ev_in[set], s_in));
    CSSM_TRY(cudaStreamWaitEvent(user, ev_in[set], 0));
    if (rc == CSSM_OK) rc = cssm_gated_forward(&c, w, plan, xd, yd, base + hl.ws, l.total, user);
    CSSM_TRY(cudaEventRecord(ev_comp[set], user));
    CSSM_TRY(cudaStreamWaitEvent(s_out, ev_comp[set], 0));
    CSSM_TRY(cudaMemcpyAsync(y_host + (size_t)b0 * per_b, yd, (size_t)cb * per_b * sizeof(float),
                             cudaMemcpyDeviceToHost, s_out));
    CSSM_TRY(cudaEventRecord(ev_out[set], s_out));
  }
  // the caller's stream observes completion of every copy
  for (int i = 0; i < 2; ++i)
    if (rc == CSSM_OK && nchunk > i) CSSM_TRY(cudaStreamWaitEvent(user, ev_out[i], 0));
  if (s_in) cudaStreamSynchronize(s_in);
  if (s_out) cudaStreamSynchronize(s_out);
  for (int i = 0; i < 2; ++i) {
    if (ev_in[i]) cudaEventDestroy(ev_in[i]);
    if (ev_comp[i]) cudaEventDestroy(ev_comp[i]);
    if (ev_out[i]) cudaEventDestroy(ev_out[i]);
  }
  if (ev_start) cudaEventDestroy(ev_start);
  if (s_in) cudaStreamDestroy(s_in);
  if (s_out) cudaStreamDestroy(s_out);
#undef CSSM_TRY
  return rc;
}

}  // extern "C"
