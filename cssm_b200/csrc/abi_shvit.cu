// C ABI of the bf16 CSSM-SHViT forward: plan (packed bf16 weights, folded BatchNorm), the two block
// kinds, the whole model on device buffers and on host buffers, and the bf16 GEMM / conv on their own.
#include <string.h>
#include <new>
#include "kernels.cuh"

namespace cssm {

static inline int packed_ld(int K) { return (K + 63) / 64 * 64; }
static inline size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

static cssm_gated_desc mixer_desc(const cssm_shvit_block_desc& d) {
  cssm_gated_desc g;
  memset(&g, 0, sizeof(g));
  g.B = d.B; g.T = d.num_timesteps; g.H = d.H; g.W = d.W; g.C = d.C;
  g.kernel_size = d.kernel_size; g.rope_mode = d.rope_mode; g.rope_base = d.rope_base;
  g.spectral_rho = d.spectral_rho; g.gate_activation = d.gate_activation;
  g.short_conv_size = d.short_conv_size; g.short_conv_spatial_size = d.short_conv_spatial_size;
  g.gate_type = d.gate_type;
  return g;
}

// The bf16 channels-last mixer path: T = 1 (the state is U_1, K_hat does not enter), no spatial
// short conv (the temporal one is a per-channel affine at T = 1 and is folded into in_proj), no
// RoPE, 14x14 or 7x7 planes.  Everything else runs the float32 block.
static bool mixer_fast(const cssm_shvit_block_desc& d) {
  return d.is_cssm && d.short_conv_spatial_size == 0 && d.rope_mode == CSSM_ROPE_NONE &&
         spectral_cl_supported(d.H, d.W, d.C, d.num_timesteps) && gemm_bf16_pick_bn(2 * d.C) != 0 &&
         gemm_bf16_pick_bn(d.C) != 0 && d.C % 64 == 0;
}

static int block_validate(const cssm_shvit_block_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->hidden <= 0) return CSSM_ERR_DIMS;
  if (d->C % 8 != 0 || d->hidden % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  if (gemm_bf16_pick_bn(d->C) == 0 || gemm_bf16_pick_bn(d->hidden) == 0) return CSSM_ERR_UNSUPPORTED;
  if (d->is_cssm) {
    if (d->num_timesteps <= 0) return CSSM_ERR_DIMS;
    if (!mixer_fast(*d)) {
      const cssm_gated_desc g = mixer_desc(*d);
      if (cssm_gated_workspace_bytes(&g) == 0) return CSSM_ERR_UNSUPPORTED;
    }
  }
  return CSSM_OK;
}

struct BlockPlan {
  size_t pw, fc1, fc2, inp, inp_bias, outp, gplan, total;   // byte offsets (unused ones = 0)
};
static BlockPlan block_plan_layout(const cssm_shvit_block_desc& d) {
  BlockPlan p;
  memset(&p, 0, sizeof(p));
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += al256(bytes); return o; };
  const size_t C = d.C, Hd = d.hidden;
  p.fc1 = take(Hd * packed_ld(d.C) * 2);
  p.fc2 = take(C * packed_ld(d.hidden) * 2);
  if (!d.is_cssm) {
    p.pw = take(C * packed_ld(d.C) * 2);
  } else if (mixer_fast(d)) {
    p.inp = take(2 * C * packed_ld(d.C) * 2);
    p.inp_bias = take(2 * C * 4 + 2 * C * 4);          // folded bias, then the column scale
    p.outp = take(C * packed_ld(d.C) * 2);
  } else {
    const cssm_gated_desc g = mixer_desc(d);
    p.gplan = take(cssm_gated_plan_bytes(&g));
  }
  p.total = off;
  return p;
}

struct BlockWs {
  size_t t, t2, hid, hid2, na, nb, ctx, maps, x32, y32, gws, total;
  size_t gws_bytes;
};
static BlockWs block_ws_layout(const cssm_shvit_block_desc& d) {
  BlockWs l;
  memset(&l, 0, sizeof(l));
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += al256(bytes); return o; };
  const size_t M = (size_t)d.B * d.H * d.W, C = d.C, Hd = d.hidden;
  l.t = take(M * C * 2);
  l.t2 = take(M * C * 2);
  const size_t hid_elems = Hd > 2 * C ? Hd : 2 * C;
  l.hid = take(M * hid_elems * 2);
  if (d.is_cssm) {
    if (d.use_dwconv) l.hid2 = take(M * Hd * 2);
    l.na = take((size_t)d.B * C * 4);
    l.nb = take((size_t)d.B * C * 4);
    if (mixer_fast(d)) {
      l.ctx = take((size_t)d.B * C * 4);
      l.maps = take((size_t)d.B * d.H * (d.W / 2 + 1) * 16);
    } else {
      const cssm_gated_desc g = mixer_desc(d);
      l.x32 = take(M * C * 4);
      l.y32 = take(M * C * 4);
      l.gws_bytes = cssm_gated_workspace_bytes(&g);
      l.gws = take(l.gws_bytes);
    }
  }
  l.total = off;
  return l;
}

// Launch trace of the call in progress on this thread (cssm_shvit_forward_timed sets it for the
// duration of its own call): before every kernel launch an event is recorded on the stream and the
// kernel kind and the algorithmic bytes of the launch (inputs + outputs + weights) are noted.
static thread_local cssm_shvit_trace* g_trace = nullptr;
static inline void trace(int kind, double bytes, cudaStream_t st) {
  cssm_shvit_trace* t = g_trace;
  if (t == nullptr || t->count >= t->capacity) return;
  cudaEventRecord(reinterpret_cast<cudaEvent_t>(t->events[t->count]), st);
  t->kinds[t->count] = kind;
  t->bytes[t->count] = bytes;
  ++t->count;
}

static int gemm_plain(const __nv_bfloat16* A, int M, int K, const __nv_bfloat16* Wt, int N, const float* bias,
                      int act, const __nv_bfloat16* res, __nv_bfloat16* out, cudaStream_t st) {
  Bf16GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.A = A; g.M = M; g.N = N; g.K = K; g.lda = K;
  g.Wt = Wt; g.ldw = packed_ld(K); g.bias = bias; g.act = act;
  g.res = res; g.ldr = N; g.out = out; g.ldo = N;
  trace(CSSM_SHVIT_K_GEMM, 2.0 * ((double)M * K + (double)M * N * (res ? 2 : 1) + (double)N * K), st);
  return launch_gemm_bf16(g, st);
}

static int conv_s2(const __nv_bfloat16* x, int B, int Hi, int Wi, int Cin, const __nv_bfloat16* Wt, int Cout,
                   const float* bias, int act, __nv_bfloat16* out, cudaStream_t st) {
  Bf16GemmArgs g;
  memset(&g, 0, sizeof(g));
  const int Ho = (Hi + 1) / 2, Wo = (Wi + 1) / 2;
  const int th = (Ho - 1) * 2 + 3 - Hi, tw = (Wo - 1) * 2 + 3 - Wi;
  g.A = x; g.M = B * Ho * Wo; g.N = Cout; g.K = 9 * Cin;
  g.ksz = 3; g.stride = 2; g.Hi = Hi; g.Wi = Wi; g.Cin = Cin; g.Ho = Ho; g.Wo = Wo;
  g.pad_h = (th > 0 ? th : 0) / 2; g.pad_w = (tw > 0 ? tw : 0) / 2;
  g.Wt = Wt; g.ldw = packed_ld(conv3x3s2_packed_k(Cin, Wi, Cout)); g.bias = bias; g.act = act;
  g.out = out; g.ldo = Cout;
  trace(CSSM_SHVIT_K_CONV_GEMM, 2.0 * ((double)B * Hi * Wi * Cin + (double)g.M * Cout + 9.0 * Cin * Cout), st);
  return launch_gemm_bf16(g, st);
}

#define CSSM_RUN(call) do { int s_ = (call); if (s_ != CSSM_OK) return s_; } while (0)

static int block_plan_init(const cssm_shvit_block_desc& d, const cssm_shvit_block_weights& w, char* plan,
                           cudaStream_t st) {
  const BlockPlan p = block_plan_layout(d);
  if (!w.norm1_scale || !w.norm1_bias || !w.norm2_scale || !w.norm2_bias || !w.fc1_kernel || !w.fc1_bias ||
      !w.fc2_kernel || !w.fc2_bias)
    return CSSM_ERR_NULL;
  CSSM_RUN(launch_pack_wt(w.fc1_kernel, d.C, d.hidden, nullptr, (__nv_bfloat16*)(plan + p.fc1), packed_ld(d.C), st));
  CSSM_RUN(launch_pack_wt(w.fc2_kernel, d.hidden, d.C, nullptr, (__nv_bfloat16*)(plan + p.fc2), packed_ld(d.hidden), st));
  if (!d.is_cssm) {
    if (!w.dw_kernel || !w.dw_bias || !w.pw_kernel || !w.pw_bias) return CSSM_ERR_NULL;
    return launch_pack_wt(w.pw_kernel, d.C, d.C, nullptr, (__nv_bfloat16*)(plan + p.pw), packed_ld(d.C), st);
  }
  if (d.use_pos_conv && (!w.dw_kernel || !w.dw_bias)) return CSSM_ERR_NULL;
  if (d.use_dwconv && (!w.mlp_dw_kernel || !w.mlp_dw_bias)) return CSSM_ERR_NULL;
  if (!w.cssm.in_proj_kernel || !w.cssm.in_proj_bias || !w.cssm.out_proj_kernel || !w.cssm.out_proj_bias)
    return CSSM_ERR_NULL;
  if (mixer_fast(d)) {
    // x_main columns of in_proj carry the T = 1 temporal conv: out[t=0] = w[k-1] * x + b (the other
    // taps meet the zero padding), so column c is scaled by w[k-1, c] and the bias becomes
    // w[k-1, c] * b_in[c] + b_t[c]; the z columns are unchanged.
    float* nb = (float*)(plan + p.inp_bias);
    float* cs = nb + 2 * d.C;
    const int k = d.short_conv_size;
    CSSM_RUN(launch_fill(cs, 2 * d.C, 1.0f, st));
    if (k > 0) {
      if (!w.cssm.conv_t_kernel || !w.cssm.conv_t_bias) return CSSM_ERR_NULL;
      const float* tap = w.cssm.conv_t_kernel + (size_t)(k - 1) * d.C;
      CSSM_RUN(launch_affine_vec(tap, nullptr, nullptr, d.C, cs, st));                      // scale[c] = tap[c]
      CSSM_RUN(launch_affine_vec(w.cssm.in_proj_bias, tap, w.cssm.conv_t_bias, d.C, nb, st));
    } else {
      CSSM_RUN(launch_affine_vec(w.cssm.in_proj_bias, nullptr, nullptr, d.C, nb, st));
    }
    CSSM_RUN(launch_affine_vec(w.cssm.in_proj_bias + d.C, nullptr, nullptr, d.C, nb + d.C, st));
    CSSM_RUN(launch_pack_wt(w.cssm.in_proj_kernel, d.C, 2 * d.C, cs, (__nv_bfloat16*)(plan + p.inp),
                            packed_ld(d.C), st));
    return launch_pack_wt(w.cssm.out_proj_kernel, d.C, d.C, nullptr, (__nv_bfloat16*)(plan + p.outp),
                          packed_ld(d.C), st);
  }
  const cssm_gated_desc g = mixer_desc(d);
  return cssm_gated_plan_init(&g, &w.cssm, plan + p.gplan, cssm_gated_plan_bytes(&g), st);
}

static int block_forward(const cssm_shvit_block_desc& d, const cssm_shvit_block_weights& w, const char* plan,
                         const __nv_bfloat16* x, __nv_bfloat16* y, char* ws, cudaStream_t st) {
  const BlockPlan p = block_plan_layout(d);
  const BlockWs l = block_ws_layout(d);
  const int M = d.B * d.H * d.W, C = d.C, Hd = d.hidden;
  __nv_bfloat16* T = (__nv_bfloat16*)(ws + l.t);
  __nv_bfloat16* X1 = (__nv_bfloat16*)(ws + l.t2);      // the residual stream after the first half
  __nv_bfloat16* HB = (__nv_bfloat16*)(ws + l.hid);
  const __nv_bfloat16* fc1 = (const __nv_bfloat16*)(plan + p.fc1);
  const __nv_bfloat16* fc2 = (const __nv_bfloat16*)(plan + p.fc2);
  if (!d.is_cssm) {
    // LN -> dw7x7 -> gelu -> Dense + residual
    trace(CSSM_SHVIT_K_LAYERNORM, 4.0 * M * C, st);
    CSSM_RUN(launch_layernorm_cl(x, w.norm1_scale, w.norm1_bias, T, M, C, st));
    trace(CSSM_SHVIT_K_DWCONV7, 4.0 * M * C, st);
    CSSM_RUN(launch_dwconv_cl(T, w.dw_kernel, w.dw_bias, nullptr, nullptr, HB, nullptr, d.B, d.H, d.W, C, 7, 0, 1, st));
    CSSM_RUN(gemm_plain(HB, M, C, (const __nv_bfloat16*)(plan + p.pw), C, w.pw_bias, 0, x, X1, st));
  } else {
    float* na = (float*)(ws + l.na);
    float* nb = (float*)(ws + l.nb);
    // LayerNorm over (T,H,W,C) of the repeated image = over (H,W,C) of the image; x + dw3x3(x)
    trace(CSSM_SHVIT_K_SAMPLE_NORM, 2.0 * M * C, st);
    CSSM_RUN(launch_sample_norm(x, w.norm1_scale, w.norm1_bias, na, nb, d.B, d.H * d.W * C, C, st));
    trace(CSSM_SHVIT_K_DWCONV3, (mixer_fast(d) ? 4.0 : 6.0) * M * C, st);
    if (mixer_fast(d)) {
      CSSM_RUN(launch_dwconv_cl(x, d.use_pos_conv ? w.dw_kernel : nullptr, w.dw_bias, na, nb, T, nullptr, d.B,
                                d.H, d.W, C, 3, 1, 0, st));
      const float* inb = (const float*)(plan + p.inp_bias);
      CSSM_RUN(gemm_plain(T, M, C, (const __nv_bfloat16*)(plan + p.inp), 2 * C, inb, 2, nullptr, HB, st));
      float* ctx = (float*)(ws + l.ctx);
      trace(CSSM_SHVIT_K_PLANE_SUM, 2.0 * M * C, st);
      CSSM_RUN(launch_plane_sum_cl(HB, 2 * C, d.B, d.H * d.W, C, ctx, st));
      GatedGateArgs ga;
      memset(&ga, 0, sizeof(ga));
      ga.ctx_sum = ctx; ga.BT = d.B; ga.C = C; ga.H = d.H; ga.W = d.W; ga.gate_type = d.gate_type;
      ga.act = d.gate_activation; ga.path = PATH_GENERIC;
      for (int i = 0; i < 6; ++i) { ga.gk[i] = w.cssm.gate_kernel[i]; ga.gb[i] = w.cssm.gate_bias[i]; }
      ga.maps = (float4*)(ws + l.maps);
      trace(CSSM_SHVIT_K_GATES, 16.0 * d.B * d.H * (d.W / 2 + 1), st);
      CSSM_RUN(launch_gated_gates(ga, st));
      trace(CSSM_SHVIT_K_SPECTRAL, 6.0 * M * C, st);          // x_main, z in; y out (bf16)
      CSSM_RUN(launch_gated_spectral_cl(HB, 2 * C, d.B, d.H, d.W, C, (const float*)(ws + l.maps), T, C, st));
      CSSM_RUN(gemm_plain(T, M, C, (const __nv_bfloat16*)(plan + p.outp), C, w.cssm.out_proj_bias, 0, x, X1, st));
    } else {
      float* x32 = (float*)(ws + l.x32);
      float* y32 = (float*)(ws + l.y32);
      CSSM_RUN(launch_dwconv_cl(x, d.use_pos_conv ? w.dw_kernel : nullptr, w.dw_bias, na, nb, nullptr, x32, d.B,
                                d.H, d.W, C, 3, 1, 0, st));
      const cssm_gated_desc g = mixer_desc(d);
      // identical frames in (x_bcast), only the last frame out
      trace(CSSM_SHVIT_K_MIXER_F32, 8.0 * M * C, st);
      CSSM_RUN(gated_forward_internal(&g, &w.cssm, plan + p.gplan, x32, y32, ws + l.gws, l.gws_bytes, st, 1, 1));
      trace(CSSM_SHVIT_K_ADD_RES, 8.0 * M * C, st);
      CSSM_RUN(launch_add_res(x, y32, X1, (long long)M * C, st));
    }
  }
  // LN -> fc1 -> gelu -> [h + dw3x3(h)] -> fc2 + residual
  trace(CSSM_SHVIT_K_LAYERNORM, 4.0 * M * C, st);
  CSSM_RUN(launch_layernorm_cl(X1, w.norm2_scale, w.norm2_bias, T, M, C, st));
  if (!(d.is_cssm && d.use_dwconv) && mlp_fused_supported(C, Hd)) {
    // fc1 + GELU + fc2 + residual in one kernel: the hidden tensor stays on chip
    trace(CSSM_SHVIT_K_MLP, 2.0 * (3.0 * M * C + 2.0 * C * Hd), st);
    return launch_mlp_fused(T, M, fc1, packed_ld(C), w.fc1_bias, fc2, packed_ld(Hd), w.fc2_bias, X1, y, st);
  }
  CSSM_RUN(gemm_plain(T, M, C, fc1, Hd, w.fc1_bias, 1, nullptr, HB, st));
  const __nv_bfloat16* h = HB;
  if (d.is_cssm && d.use_dwconv) {
    __nv_bfloat16* H2 = (__nv_bfloat16*)(ws + l.hid2);
    trace(CSSM_SHVIT_K_DWCONV3, 4.0 * M * Hd, st);
    CSSM_RUN(launch_dwconv_cl(HB, w.mlp_dw_kernel, w.mlp_dw_bias, nullptr, nullptr, H2, nullptr, d.B, d.H, d.W, Hd,
                              3, 1, 0, st));
    h = H2;
  }
  return gemm_plain(h, M, Hd, fc2, C, w.fc2_bias, 0, X1, y, st);
}

// ---------------------------------------------------------------------------- model ----
static int model_validate(const cssm_shvit_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->H <= 0 || d->W <= 0 || d->Cin <= 0 || d->num_classes <= 0) return CSSM_ERR_DIMS;
  int nb = 0;
  for (int s = 0; s < 4; ++s) {
    if (d->embed_dims[s] <= 0 || d->depths[s] <= 0) return CSSM_ERR_DIMS;
    if (d->embed_dims[s] % 32 != 0) return CSSM_ERR_UNSUPPORTED;
    nb += d->depths[s];
  }
  if (nb > CSSM_SHVIT_MAX_BLOCKS) return CSSM_ERR_SIZE_LIMIT;
  if (d->Cin > 16 || (d->embed_dims[0] / 2) % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

static cssm_shvit_block_desc stage_block_desc(const cssm_shvit_desc& d, int s, int H, int W) {
  cssm_shvit_block_desc b;
  memset(&b, 0, sizeof(b));
  b.B = d.B; b.H = H; b.W = W; b.C = d.embed_dims[s];
  b.is_cssm = d.use_cssm[s] ? 1 : 0;
  b.hidden = (int)((float)d.embed_dims[s] * d.mlp_ratio);
  b.num_timesteps = d.num_timesteps; b.kernel_size = d.kernel_sizes[s];
  b.use_pos_conv = d.use_pos_conv; b.use_dwconv = d.use_dwconv;
  b.rope_mode = d.rope_mode; b.rope_base = d.rope_base; b.spectral_rho = d.spectral_rho;
  b.gate_activation = d.gate_activation; b.short_conv_size = d.short_conv_size;
  b.short_conv_spatial_size = d.short_conv_spatial_size; b.gate_type = d.gate_type;
  return b;
}

struct ModelPlan {
  size_t c1w, c1b, c2w, c2b, dsw[3], dsb[3], blocks[CSSM_SHVIT_MAX_BLOCKS], scratch, total;
};
struct ModelWs { size_t a, b, pooled, blk, total; size_t blk_bytes; };

// Walks the stages once: sizes of the plan / workspace, and the per-block descriptors.
struct ModelWalk {
  ModelPlan plan; ModelWs ws;
  cssm_shvit_block_desc bd[CSSM_SHVIT_MAX_BLOCKS];
  int stage_of[CSSM_SHVIT_MAX_BLOCKS];
  int nblocks; int status;
  int Hs[4], Ws[4];
};
static ModelWalk model_walk(const cssm_shvit_desc& d) {
  ModelWalk m;
  memset(&m, 0, sizeof(m));
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += al256(bytes); return o; };
  const int E0 = d.embed_dims[0];
  m.plan.c1w = take((size_t)9 * d.Cin * (E0 / 2) * 4);
  m.plan.c1b = take((size_t)(E0 / 2) * 4);
  m.plan.c2w = take((size_t)E0 * packed_ld(conv3x3s2_packed_k(E0 / 2, (d.W + 1) / 2, E0)) * 2);
  m.plan.c2b = take((size_t)E0 * 4);
  int H = (((d.H + 1) / 2) + 1) / 2, W = (((d.W + 1) / 2) + 1) / 2;
  int Wprev = W;                                       // width of the input of the next downsample conv
  size_t act_max = (size_t)d.B * ((d.H + 1) / 2) * ((d.W + 1) / 2) * (E0 / 2);
  size_t blk_ws = 0;
  for (int s = 0; s < 4; ++s) {
    if (s > 0) {
      m.plan.dsw[s - 1] = take((size_t)d.embed_dims[s] * packed_ld(conv3x3s2_packed_k(d.embed_dims[s - 1], Wprev, d.embed_dims[s])) * 2);
      m.plan.dsb[s - 1] = take((size_t)d.embed_dims[s] * 4);
      H = (H + 1) / 2; W = (W + 1) / 2;
      Wprev = W;
    }
    m.Hs[s] = H; m.Ws[s] = W;
    const size_t act = (size_t)d.B * H * W * d.embed_dims[s];
    if (act > act_max) act_max = act;
    for (int b = 0; b < d.depths[s]; ++b) {
      cssm_shvit_block_desc bd = stage_block_desc(d, s, H, W);
      const int st = block_validate(&bd);
      if (st != CSSM_OK && m.status == CSSM_OK) m.status = st;
      if (st == CSSM_OK) {
        m.plan.blocks[m.nblocks] = take(block_plan_layout(bd).total);
        const size_t wsb = block_ws_layout(bd).total;
        if (wsb > blk_ws) blk_ws = wsb;
      }
      m.bd[m.nblocks] = bd;
      m.stage_of[m.nblocks] = s;
      ++m.nblocks;
    }
  }
  int cmax = 0;
  for (int s = 0; s < 4; ++s) cmax = d.embed_dims[s] > cmax ? d.embed_dims[s] : cmax;
  m.plan.scratch = take((size_t)2 * cmax * 4);      // BatchNorm scale / bias during plan_init
  m.plan.total = off;
  size_t wo = 0;
  auto wtake = [&](size_t bytes) { const size_t o = wo; wo += al256(bytes); return o; };
  m.ws.a = wtake(act_max * 2);
  m.ws.b = wtake(act_max * 2);
  m.ws.pooled = wtake((size_t)d.B * d.embed_dims[3] * 4);
  m.ws.blk = wtake(blk_ws);
  m.ws.blk_bytes = blk_ws;
  m.ws.total = wo;
  return m;
}

static int model_forward(const cssm_shvit_desc& d, const cssm_shvit_weights& w, const char* plan,
                         const __nv_bfloat16* x, float* logits, char* ws, cudaStream_t st) {
  const ModelWalk m = model_walk(d);
  __nv_bfloat16* A = (__nv_bfloat16*)(ws + m.ws.a);
  __nv_bfloat16* B = (__nv_bfloat16*)(ws + m.ws.b);
  const int E0 = d.embed_dims[0];
  const int H1 = (d.H + 1) / 2, W1 = (d.W + 1) / 2;
  // patch embed: ConvBN -> gelu -> ConvBN
  trace(CSSM_SHVIT_K_STEM_CONV, 2.0 * ((double)d.B * d.H * d.W * d.Cin + (double)d.B * H1 * W1 * (E0 / 2)), st);
  CSSM_RUN(launch_stem_conv1(x, (const float*)(plan + m.plan.c1w), (const float*)(plan + m.plan.c1b), A, d.B, d.H,
                             d.W, d.Cin, E0 / 2, 1, st));
  CSSM_RUN(conv_s2(A, d.B, H1, W1, E0 / 2, (const __nv_bfloat16*)(plan + m.plan.c2w), E0,
                   (const float*)(plan + m.plan.c2b), 0, B, st));
  __nv_bfloat16* cur = B;
  __nv_bfloat16* other = A;
  int bi = 0;
  for (int s = 0; s < 4; ++s) {
    if (s > 0) {
      CSSM_RUN(conv_s2(cur, d.B, m.Hs[s - 1], m.Ws[s - 1], d.embed_dims[s - 1],
                       (const __nv_bfloat16*)(plan + m.plan.dsw[s - 1]), d.embed_dims[s],
                       (const float*)(plan + m.plan.dsb[s - 1]), 0, other, st));
      __nv_bfloat16* t = cur; cur = other; other = t;
    }
    for (int b = 0; b < d.depths[s]; ++b, ++bi) {
      CSSM_RUN(block_forward(m.bd[bi], w.blocks[bi], plan + m.plan.blocks[bi], cur, other, ws + m.ws.blk, st));
      __nv_bfloat16* t = cur; cur = other; other = t;
    }
  }
  const int C3 = d.embed_dims[3], P3 = m.Hs[3] * m.Ws[3];
  trace(CSSM_SHVIT_K_LAYERNORM, 4.0 * d.B * P3 * C3, st);
  CSSM_RUN(launch_layernorm_cl(cur, w.norm_scale, w.norm_bias, other, (long long)d.B * P3, C3, st));
  float* pooled = (float*)(ws + m.ws.pooled);
  trace(CSSM_SHVIT_K_POOL, 2.0 * d.B * P3 * C3, st);
  CSSM_RUN(launch_pool_cl(other, d.B, P3, C3, d.head_pool == 0 ? 1 : 0, pooled, st));
  trace(CSSM_SHVIT_K_HEAD, 4.0 * ((double)d.B * C3 + (double)d.B * d.num_classes + (double)C3 * d.num_classes), st);
  CSSM_RUN(launch_head(pooled, w.head_kernel, w.head_bias, logits, d.B, C3, d.num_classes, st));
  trace(CSSM_SHVIT_K_END, 0.0, st);
  return CSSM_OK;
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_shvit_block_plan_bytes(const cssm_shvit_block_desc* d) {
  if (block_validate(d) != CSSM_OK) return 0;
  return block_plan_layout(*d).total;
}
size_t cssm_shvit_block_workspace_bytes(const cssm_shvit_block_desc* d) {
  if (block_validate(d) != CSSM_OK) return 0;
  return block_ws_layout(*d).total;
}
int cssm_shvit_block_plan_init(const cssm_shvit_block_desc* d, const cssm_shvit_block_weights* w, void* plan,
                               size_t plan_bytes, void* stream) {
  int s = block_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  if (plan_bytes < block_plan_layout(*d).total) return CSSM_ERR_WORKSPACE;
  return block_plan_init(*d, *w, (char*)plan, (cudaStream_t)stream);
}
int cssm_shvit_block_forward(const cssm_shvit_block_desc* d, const cssm_shvit_block_weights* w, const void* plan,
                             const void* x_bf16, void* y_bf16, void* workspace, size_t workspace_bytes,
                             void* stream) {
  int s = block_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan || !x_bf16 || !y_bf16 || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(plan) || !aligned16(x_bf16) || !aligned16(y_bf16) || !aligned16(workspace)) return CSSM_ERR_ALIGN;
  if (workspace_bytes < block_ws_layout(*d).total) return CSSM_ERR_WORKSPACE;
  return block_forward(*d, *w, (const char*)plan, (const __nv_bfloat16*)x_bf16, (__nv_bfloat16*)y_bf16,
                       (char*)workspace, (cudaStream_t)stream);
}

size_t cssm_shvit_plan_bytes(const cssm_shvit_desc* d) {
  if (model_validate(d) != CSSM_OK) return 0;
  const ModelWalk m = model_walk(*d);
  return m.status == CSSM_OK ? m.plan.total : 0;
}
size_t cssm_shvit_workspace_bytes(const cssm_shvit_desc* d) {
  if (model_validate(d) != CSSM_OK) return 0;
  const ModelWalk m = model_walk(*d);
  return m.status == CSSM_OK ? m.ws.total : 0;
}
int cssm_shvit_plan_init(const cssm_shvit_desc* d, const cssm_shvit_weights* w, void* plan, size_t plan_bytes,
                         void* stream) {
  int s = model_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  const ModelWalk m = model_walk(*d);
  if (m.status != CSSM_OK) return m.status;
  if (plan_bytes < m.plan.total) return CSSM_ERR_WORKSPACE;
  if (!w->norm_scale || !w->norm_bias || !w->head_kernel || !w->head_bias) return CSSM_ERR_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  char* pl = (char*)plan;
  float* sc = (float*)(pl + m.plan.scratch);
  int cmax = 0;
  for (int i = 0; i < 4; ++i) cmax = d->embed_dims[i] > cmax ? d->embed_dims[i] : cmax;
  const int E0 = d->embed_dims[0];
  auto fold = [&](const cssm_shvit_convbn& c, int Cout, float* bias_out) -> int {
    if (!c.kernel || !c.bn_scale || !c.bn_bias || !c.bn_mean || !c.bn_var) return CSSM_ERR_NULL;
    return launch_bn_fold(c.bn_scale, c.bn_bias, c.bn_mean, c.bn_var, Cout, sc, bias_out, st);
  };
  // first conv: float32 (9*Cin, Cout) kernel scaled by the BatchNorm factor
  CSSM_RUN(fold(w->patch[0], E0 / 2, (float*)(pl + m.plan.c1b)));
  CSSM_RUN(launch_scale_cols(w->patch[0].kernel, 9 * d->Cin, E0 / 2, sc, (float*)(pl + m.plan.c1w), st));
  CSSM_RUN(fold(w->patch[1], E0, (float*)(pl + m.plan.c2b)));
  CSSM_RUN(launch_pack_conv3x3(w->patch[1].kernel, E0 / 2, E0, (d->W + 1) / 2, sc,
                               (__nv_bfloat16*)(pl + m.plan.c2w), st));
  for (int i = 1; i < 4; ++i) {
    CSSM_RUN(fold(w->down[i - 1], d->embed_dims[i], (float*)(pl + m.plan.dsb[i - 1])));
    CSSM_RUN(launch_pack_conv3x3(w->down[i - 1].kernel, d->embed_dims[i - 1], d->embed_dims[i], m.Ws[i - 1], sc,
                                 (__nv_bfloat16*)(pl + m.plan.dsw[i - 1]), st));
  }
  for (int b = 0; b < m.nblocks; ++b)
    CSSM_RUN(block_plan_init(m.bd[b], w->blocks[b], pl + m.plan.blocks[b], st));
  return CSSM_OK;
}
int cssm_shvit_forward(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan, const void* x_bf16,
                       float* logits, void* workspace, size_t workspace_bytes, void* stream) {
  int s = model_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !plan || !x_bf16 || !logits || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(plan) || !aligned16(x_bf16) || !aligned16(logits) || !aligned16(workspace)) return CSSM_ERR_ALIGN;
  const ModelWalk m = model_walk(*d);
  if (m.status != CSSM_OK) return m.status;
  if (workspace_bytes < m.ws.total) return CSSM_ERR_WORKSPACE;
  return model_forward(*d, *w, (const char*)plan, (const __nv_bfloat16*)x_bf16, logits, (char*)workspace,
                       (cudaStream_t)stream);
}

int cssm_shvit_forward_timed(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                             const void* x_bf16, float* logits, void* workspace, size_t workspace_bytes,
                             void* stream, cssm_shvit_trace* tr) {
  if (!tr || !tr->events || !tr->kinds || !tr->bytes || tr->capacity <= 0) return CSSM_ERR_NULL;
  tr->count = 0;
  g_trace = tr;
  const int s = cssm_shvit_forward(d, w, plan, x_bf16, logits, workspace, workspace_bytes, stream);
  g_trace = nullptr;
  return s;
}

// Host-buffer entry point: the batch is cut into chunks; the host->device copy of chunk k+1 runs on
// a second stream while chunk k computes (two staging buffers, ordered by events), one device->host
// copy of all logits and one wait at the end.
static int host_chunks(int B) { return (B >= 256 && B % 4 == 0) ? 4 : ((B >= 64 && B % 2 == 0) ? 2 : 1); }
struct HostWs { size_t model, xbuf[2], logits, total; size_t model_bytes; int chunk_b; };
static HostWs host_ws_layout(const cssm_shvit_desc& d) {
  HostWs h;
  memset(&h, 0, sizeof(h));
  cssm_shvit_desc c = d;
  h.chunk_b = d.B / host_chunks(d.B);
  c.B = h.chunk_b;
  h.model_bytes = cssm_shvit_workspace_bytes(&c);
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += al256(bytes); return o; };
  h.model = take(h.model_bytes);
  const size_t xb = (size_t)h.chunk_b * d.H * d.W * d.Cin * 2;
  h.xbuf[0] = take(xb);
  h.xbuf[1] = take(xb);
  h.logits = take((size_t)d.B * d.num_classes * 4);
  h.total = off;
  return h;
}

size_t cssm_shvit_host_workspace_bytes(const cssm_shvit_desc* d) {
  if (cssm_shvit_workspace_bytes(d) == 0) return 0;
  return host_ws_layout(*d).total;
}
int cssm_shvit_forward_host(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                            const void* x_bf16_host, float* logits_host, void* workspace, size_t workspace_bytes,
                            void* stream) {
  if (cssm_shvit_workspace_bytes(d) == 0) return model_validate(d) != CSSM_OK ? model_validate(d) : CSSM_ERR_UNSUPPORTED;
  if (!w || !plan || !x_bf16_host || !logits_host || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(workspace) || !aligned16(plan)) return CSSM_ERR_ALIGN;
  const HostWs h = host_ws_layout(*d);
  if (workspace_bytes < h.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  const int nchunk = d->B / h.chunk_b;
  const size_t xb = (size_t)h.chunk_b * d->H * d->W * d->Cin * 2;
  float* ld = (float*)(ws + h.logits);
  cssm_shvit_desc c = *d;
  c.B = h.chunk_b;
  cudaStream_t sc = nullptr;
  cudaEvent_t ev_start = nullptr, ev_in[2] = {nullptr, nullptr}, ev_comp[2] = {nullptr, nullptr};
  int rc = CSSM_OK;
  cudaError_t e = cudaSuccess;
#define CSSM_TRY(call) do { if (rc == CSSM_OK) { e = (call); if (e != cudaSuccess) { set_cuda_error(e); rc = CSSM_ERR_CUDA; } } } while (0)
  CSSM_TRY(cudaStreamCreateWithFlags(&sc, cudaStreamNonBlocking));
  CSSM_TRY(cudaEventCreateWithFlags(&ev_start, cudaEventDisableTiming));
  for (int i = 0; i < 2; ++i) {
    CSSM_TRY(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
    CSSM_TRY(cudaEventCreateWithFlags(&ev_comp[i], cudaEventDisableTiming));
  }
  // copies start only after work already queued on the caller's stream (e.g. plan_init)
  CSSM_TRY(cudaEventRecord(ev_start, st));
  CSSM_TRY(cudaStreamWaitEvent(sc, ev_start, 0));
  for (int k = 0; k < nchunk && rc == CSSM_OK; ++k) {
    const int j = k & 1;
    if (k >= 2) CSSM_TRY(cudaStreamWaitEvent(sc, ev_comp[j], 0));      // chunk k-2 has left this buffer
    CSSM_TRY(cudaMemcpyAsync(ws + h.xbuf[j], (const char*)x_bf16_host + (size_t)k * xb, xb,
                             cudaMemcpyHostToDevice, sc));
    CSSM_TRY(cudaEventRecord(ev_in[j], sc));
    CSSM_TRY(cudaStreamWaitEvent(st, ev_in[j], 0));
    if (rc == CSSM_OK)
      rc = cssm_shvit_forward(&c, w, plan, ws + h.xbuf[j], ld + (size_t)k * h.chunk_b * d->num_classes,
                              ws + h.model, h.model_bytes, stream);
    CSSM_TRY(cudaEventRecord(ev_comp[j], st));
  }
  CSSM_TRY(cudaMemcpyAsync(logits_host, ld, (size_t)d->B * d->num_classes * 4, cudaMemcpyDeviceToHost, st));
  // always drain both streams before the events and the stream are destroyed
  cudaError_t e1 = cudaStreamSynchronize(st), e2 = sc ? cudaStreamSynchronize(sc) : cudaSuccess;
  if (rc == CSSM_OK && (e1 != cudaSuccess || e2 != cudaSuccess)) {
    set_cuda_error(e1 != cudaSuccess ? e1 : e2);
    rc = CSSM_ERR_CUDA;
  }
#undef CSSM_TRY
  for (int i = 0; i < 2; ++i) {
    if (ev_in[i]) cudaEventDestroy(ev_in[i]);
    if (ev_comp[i]) cudaEventDestroy(ev_comp[i]);
  }
  if (ev_start) cudaEventDestroy(ev_start);
  if (sc) cudaStreamDestroy(sc);
  return rc;
}

// ---- streaming host entry point: the next batch's images are copied while this one computes ----
struct PipeWs { size_t model, xbuf[2], logits, total; size_t model_bytes, xbytes; };
static PipeWs pipe_ws_layout(const cssm_shvit_desc& d) {
  PipeWs h;
  memset(&h, 0, sizeof(h));
  h.model_bytes = cssm_shvit_workspace_bytes(&d);
  h.xbytes = (size_t)d.B * d.H * d.W * d.Cin * 2;
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += al256(bytes); return o; };
  h.model = take(h.model_bytes);
  h.xbuf[0] = take(h.xbytes);
  h.xbuf[1] = take(h.xbytes);
  h.logits = take((size_t)d.B * d.num_classes * 4);
  h.total = off;
  return h;
}

}  // extern "C"
extern "C" {

int cssm_host_pipe_create(cssm_host_pipe** pipe) {
  if (!pipe) return CSSM_ERR_NULL;
  *pipe = nullptr;
  cssm_host_pipe* p = new (std::nothrow) cssm_host_pipe();
  if (!p) return CSSM_ERR_CUDA;
  memset(p, 0, sizeof(*p));
  cudaError_t e = cudaStreamCreateWithFlags(&p->copy, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&p->copied[i], cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->computed, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    set_cuda_error(e);
    cssm_host_pipe_destroy(p);
    return CSSM_ERR_CUDA;
  }
  *pipe = p;
  return CSSM_OK;
}

int cssm_host_pipe_destroy(cssm_host_pipe* p) {
  if (!p) return CSSM_OK;
  if (p->copy) cudaStreamSynchronize(p->copy);        // a prefetch may still be reading the host buffer
  for (int i = 0; i < 2; ++i)
    if (p->copied[i]) cudaEventDestroy(p->copied[i]);
  if (p->computed) cudaEventDestroy(p->computed);
  if (p->copy) cudaStreamDestroy(p->copy);
  delete p;
  return CSSM_OK;
}

size_t cssm_shvit_host_pipe_workspace_bytes(const cssm_shvit_desc* d) {
  if (cssm_shvit_workspace_bytes(d) == 0) return 0;
  return pipe_ws_layout(*d).total;
}

int cssm_shvit_forward_host_pipelined(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                                      cssm_host_pipe* p, const void* x_bf16_host,
                                      const void* x_next_bf16_host, float* logits_host, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  if (cssm_shvit_workspace_bytes(d) == 0) return model_validate(d) != CSSM_OK ? model_validate(d) : CSSM_ERR_UNSUPPORTED;
  if (!w || !plan || !p || !x_bf16_host || !logits_host || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(workspace) || !aligned16(plan)) return CSSM_ERR_ALIGN;
  const PipeWs h = pipe_ws_layout(*d);
  if (workspace_bytes < h.total) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  int j = 0;
  int rc = host_pipe_stage(p, workspace, ws + h.xbuf[0], ws + h.xbuf[1], h.xbytes, x_bf16_host,
                           x_next_bf16_host, st, &j);
  float* ld = (float*)(ws + h.logits);
  if (rc == CSSM_OK)
    rc = cssm_shvit_forward(d, w, plan, ws + h.xbuf[j], ld, ws + h.model, h.model_bytes, stream);
  if (rc == CSSM_OK) {
    const cudaError_t e = cudaMemcpyAsync(logits_host, ld, (size_t)d->B * d->num_classes * 4,
                                          cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) { set_cuda_error(e); rc = CSSM_ERR_CUDA; }
  }
  const cudaError_t e1 = cudaStreamSynchronize(st);
  if (rc == CSSM_OK && e1 != cudaSuccess) { set_cuda_error(e1); rc = CSSM_ERR_CUDA; }
  if (rc != CSSM_OK) host_pipe_abort(p);
  return rc;
}

int32_t cssm_bf16_packed_ld(int32_t K) { return packed_ld(K); }
int cssm_bf16_pack_weight(const float* kernel, int32_t K, int32_t N, const float* col_scale, void* wt,
                          void* stream) {
  if (!kernel || !wt) return CSSM_ERR_NULL;
  if (K <= 0 || N <= 0) return CSSM_ERR_DIMS;
  return launch_pack_wt(kernel, K, N, col_scale, (__nv_bfloat16*)wt, packed_ld(K), (cudaStream_t)stream);
}
int cssm_bf16_gemm(const void* A, int32_t M, int32_t K, const void* wt, int32_t N, const float* bias, int32_t act,
                   const void* res, void* out, void* stream) {
  if (!A || !wt || !out) return CSSM_ERR_NULL;
  return gemm_plain((const __nv_bfloat16*)A, M, K, (const __nv_bfloat16*)wt, N, bias, act,
                    (const __nv_bfloat16*)res, (__nv_bfloat16*)out, (cudaStream_t)stream);
}
int cssm_bf16_mlp(const void* a, int32_t M, int32_t C, int32_t Hd, const void* w1t, const float* b1,
                  const void* w2t, const float* b2, const void* res, void* out, void* stream) {
  if (M <= 0 || C <= 0 || Hd <= 0) return CSSM_ERR_DIMS;
  if (!mlp_fused_supported(C, Hd)) return CSSM_ERR_UNSUPPORTED;
  return launch_mlp_fused((const __nv_bfloat16*)a, M, (const __nv_bfloat16*)w1t, packed_ld(C), b1,
                          (const __nv_bfloat16*)w2t, packed_ld(Hd), b2, (const __nv_bfloat16*)res,
                          (__nv_bfloat16*)out, (cudaStream_t)stream);
}
int32_t cssm_bf16_conv3x3s2_packed_ld(int32_t Cin, int32_t Wi, int32_t Cout) { return packed_ld(conv3x3s2_packed_k(Cin, Wi, Cout)); }
int cssm_bf16_pack_conv3x3s2_weight(const float* kernel, int32_t Cin, int32_t Cout, int32_t Wi,
                                    const float* col_scale, void* wt, void* stream) {
  if (!kernel || !wt) return CSSM_ERR_NULL;
  if (Cin <= 0 || Cout <= 0 || Wi <= 0) return CSSM_ERR_DIMS;
  return launch_pack_conv3x3(kernel, Cin, Cout, Wi, col_scale, (__nv_bfloat16*)wt, (cudaStream_t)stream);
}
int cssm_bf16_conv3x3s2(const void* x, int32_t B, int32_t Hi, int32_t Wi, int32_t Cin, const void* wt,
                        int32_t Cout, const float* bias, int32_t act, void* out, void* stream) {
  if (!x || !wt || !out) return CSSM_ERR_NULL;
  if (B <= 0 || Hi <= 0 || Wi <= 0 || Cin <= 0 || Cout <= 0) return CSSM_ERR_DIMS;
  return conv_s2((const __nv_bfloat16*)x, B, Hi, Wi, Cin, (const __nv_bfloat16*)wt, Cout, bias, act,
                 (__nv_bfloat16*)out, (cudaStream_t)stream);
}

}  // extern "C"
