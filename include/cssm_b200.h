/*
 * cssm_b200 — C ABI of the B200 (sm_100a) forward pass of CSSM's spectral SSM blocks.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void* so the header needs no CUDA include).  Ownership: the caller allocates every
 * input, output, plan and workspace buffer; the library never allocates, frees or keeps
 * a pointer after the call returns.  All work is enqueued on the caller's stream; no
 * call synchronises the device.  Every function returns a cssm_status (0 = ok) and never
 * throws, aborts or traps.  Activations and weights are float32.
 *
 * The reference interface each entry point stands in for is cited by file:line of
 * drewlinsley/CSSM (src/models/cssm.py unless another file is named).
 */
#ifndef CSSM_B200_H_
#define CSSM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cssm_status {
  CSSM_OK = 0,
  CSSM_ERR_NULL = 1,        /* a required pointer is NULL                               */
  CSSM_ERR_DIMS = 2,        /* a dimension is zero, negative or inconsistent            */
  CSSM_ERR_UNSUPPORTED = 3, /* a field combination this build has no kernel for         */
  CSSM_ERR_ALIGN = 4,       /* a pointer is not 16-byte aligned                         */
  CSSM_ERR_WORKSPACE = 5,   /* plan or workspace buffer too small                       */
  CSSM_ERR_CUDA = 6,        /* a CUDA runtime call or launch failed (see cssm_last_cuda_error) */
  CSSM_ERR_SIZE_LIMIT = 7   /* size beyond a documented fixed maximum                   */
} cssm_status;

typedef enum cssm_rope_mode {      /* apply_rope modes, cssm.py:94-262 */
  CSSM_ROPE_NONE = 0,
  CSSM_ROPE_SPATIOTEMPORAL = 1,
  CSSM_ROPE_TEMPORAL = 2,
  CSSM_ROPE_SPATIAL_ONLY = 3,
  CSSM_ROPE_MROPE = 4
} cssm_rope_mode;

/* CSSM_GATE_CHANNEL (per-channel / per-head decay scalars, 1x1-conv spatial input gates) exists for
   the DeltaNet and GDN blocks, CSSM_GATE_SCALAR (one scalar per frame and gate) for the GDN block;
   the other blocks reject them. */
typedef enum cssm_gate_type { CSSM_GATE_DENSE = 0, CSSM_GATE_FACTORED = 1, CSSM_GATE_CHANNEL = 2,
                              CSSM_GATE_SCALAR = 3 } cssm_gate_type;

typedef enum cssm_gate_act {       /* GatedCSSM._compute_gate, cssm.py:432-441 */
  CSSM_ACT_SOFTPLUS = 0,
  CSSM_ACT_SIGMOID2 = 1,
  CSSM_ACT_EXP_CLIP = 2
} cssm_gate_act;

const char* cssm_strerror(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* cssm_last_cuda_error(void);
/* "cssm_b200 <version> sm_100a" */
const char* cssm_version(void);

/* ------------------------------------------------------------------ GatedCSSM --- */
/* Fields of the Flax dataclass GatedCSSM (cssm.py:416-430) that the depthwise path
 * reads, plus the call-time shape of x (cssm.py:455-456). */
typedef struct cssm_gated_desc {
  int32_t B, T, H, W, C;
  int32_t kernel_size;              /* spectral kernel is (C, ks, ks)                   */
  int32_t rope_mode;                /* cssm_rope_mode                                   */
  float   rope_base;
  float   spectral_rho;
  int32_t gate_activation;          /* cssm_gate_act                                    */
  int32_t short_conv_size;          /* temporal causal taps, 0 = layer absent           */
  int32_t short_conv_spatial_size;  /* spatial depthwise k, 0 = layer absent            */
  int32_t gate_type;                /* cssm_gate_type                                   */
} cssm_gated_desc;

/* Parameter tree of GatedCSSM in Flax layout (cssm.py:481-584): Dense kernels are
 * (in, out) row-major, conv kernels HWIO.  gate_* order: delta_proj, B_proj, C_proj;
 * for factored gates index 2*g is "<name>_h" (C,H) and 2*g+1 is "<name>_w" (C,W/2+1),
 * for dense gates index g is "<name>" (C, H*(W/2+1)) and entries 3..5 are ignored. */
typedef struct cssm_gated_weights {
  const float* in_proj_kernel;   /* (C, 2C)   */
  const float* in_proj_bias;     /* (2C)      */
  const float* conv_sp_kernel;   /* (k,k,1,C) or NULL when short_conv_spatial_size==0 */
  const float* conv_sp_bias;     /* (C)       */
  const float* conv_t_kernel;    /* (k,1,C)   or NULL when short_conv_size==0         */
  const float* conv_t_bias;      /* (C)       */
  const float* kernel;           /* (C,ks,ks) */
  const float* gate_kernel[6];
  const float* gate_bias[6];
  const float* out_proj_kernel;  /* (C, C)    */
  const float* out_proj_bias;    /* (C)       */
} cssm_gated_weights;

/* Bytes of the weight-derived plan (squashed kernel spectrum K_hat, RoPE tables) and of
 * the per-call workspace.  Both return 0 for a descriptor the library rejects. */
size_t cssm_gated_plan_bytes(const cssm_gated_desc* d);
size_t cssm_gated_workspace_bytes(const cssm_gated_desc* d);

/* Weight-only precompute: centred pad of `kernel` to (H,W), rfft2,
 * K*rho/(1+|K|), GOOM magnitude floor; RoPE cos/sin tables.
 * Replaces cssm.py:505-529 (+ :29-46, goom.py:161-173) and the angle tables of
 * apply_rope (cssm.py:121-248).  Call again whenever `kernel` changes. */
int cssm_gated_plan_init(const cssm_gated_desc* d, const cssm_gated_weights* w,
                         void* plan, size_t plan_bytes, void* stream);

/* Whole block: y = GatedCSSM(x), x and y (B,T,H,W,C) float32 on the device.
 * Replaces GatedCSSM.__call__ -> _forward_depthwise, cssm.py:443-474, 476-585. */
int cssm_gated_forward(const cssm_gated_desc* d, const cssm_gated_weights* w,
                       const void* plan, const float* x, float* y,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Last-frame-only variant: y_last (B,H,W,C) = GatedCSSM(x)[:, -1].  For callers that read only
 * the final frame of a depth-1 stack (SimpleCSSM with frame_readout='last' takes x[:, -1] right
 * after the block, src/models/simple_cssm.py:482, 524-526; CSSMSHViTBlock takes x[:, -1],
 * src/models/cssm_shvit.py:214).  The recurrence still runs over all T steps; the inverse
 * transforms, the SiLU(z) gate, the stores and the out_proj of the earlier frames are skipped.
 * Same plan and workspace as cssm_gated_forward. */
int cssm_gated_forward_last(const cssm_gated_desc* d, const cssm_gated_weights* w,
                            const void* plan, const float* x, float* y_last,
                            void* workspace, size_t workspace_bytes, void* stream);

/* bf16 activations, fp32 weights (the mixers of CSSM-SHViT run inside a bf16 model: src/models/
 * cssm_shvit.py:150-214): x is bfloat16 (B,T,H,W,C).  GatedCSSM has no dtype field, so with fp32
 * parameters Flax promotes its Dense / FFT arithmetic AND its result to float32 (src/models/cssm.py:
 * 416-430, 480-585); this entry point does the same: it widens x, runs the fp32 block and writes y
 * as float32 (y_is_bf16 = 0, the reference's behaviour) or rounded to bfloat16 (y_is_bf16 = 1, for
 * callers that keep a bf16 residual stream).  Tolerance against the fp64 oracle on the same bf16
 * input: rel-L2 <= 1e-4 for the float32 result, <= 2e-2 for the bfloat16 one. */
size_t cssm_gated_bf16_workspace_bytes(const cssm_gated_desc* d);
int cssm_gated_forward_bf16(const cssm_gated_desc* d, const cssm_gated_weights* w,
                            const void* plan, const void* x_bf16, void* y, int32_t y_is_bf16,
                            void* workspace, size_t workspace_bytes, void* stream);

/* Same block with x and y in HOST memory (pinned memory gives the overlap): the batch is
 * cut into chunks whose host->device copy, kernels and device->host copy overlap on
 * three streams ordered by events.  `workspace` must hold
 * cssm_gated_host_workspace_bytes(d, chunk_b) bytes of DEVICE memory.  Synchronises the
 * internal streams with `stream` before returning control (the call itself is still
 * asynchronous with respect to the host only until its final event wait). */
size_t cssm_gated_host_workspace_bytes(const cssm_gated_desc* d, int32_t chunk_b);
int cssm_gated_forward_host(const cssm_gated_desc* d, const cssm_gated_weights* w,
                            const void* plan, const float* x_host, float* y_host,
                            int32_t chunk_b, void* workspace, size_t workspace_bytes,
                            void* stream);

/* ---- stages of the gated block, exposed for tests, profiling and partial drop-in ---- */

/* RoPE + in_proj: xz[(bt*2C + n)*H*W + hw] = sum_c rope(x)[bt,hw,c] * Wk[c,n] + b[n].
 * Planes 0..C-1 of each frame are x_main; planes C..2C-1 hold silu(z) (the SiLU of the
 * output gate, cssm.py:581, is applied where z is produced).  cssm.py:462-463, 480-484. */
int cssm_gated_in_proj(const cssm_gated_desc* d, const cssm_gated_weights* w,
                       const void* plan, const float* x, float* xz_planar, void* stream);

/* Spatial depthwise conv + causal temporal conv + SiLU on the x_main planes, in place,
 * and the per-plane sums that give ctx.  cssm.py:487-502, 536.
 * ctx_sum is (B*T, C); divide by H*W for the mean. */
int cssm_gated_short_conv(const cssm_gated_desc* d, const cssm_gated_weights* w,
                          float* xz_planar, float* ctx_sum, void* stream);

/* Gate maps from ctx: per (b,t) and frequency bin the four floats
 * {exp(-Delta), (Delta+1e-8)*B, C/(H*W), 1e-7*(Delta+1e-8)}.  cssm.py:538-567.
 * The bin order inside a (b,t) map is internal to the library. */
int cssm_gated_gates(const cssm_gated_desc* d, const cssm_gated_weights* w,
                     const float* ctx_sum, float* gate_maps, void* stream);

/* Fused spectral kernel: for each (b,c): for t: rfft2(x_main[b,t,c]),
 * h = K_hat*exp(-Delta)*h + (Delta+1e-8)*floor(B*X), y = irfft2(C*h) * (stored silu(z))[b,t,c];
 * y overwrites the x_main plane.  The state h never leaves the SM.
 * Replaces cssm.py:532-533, 558-581 (rfft2, to_goom, associative_scan of
 * math.py:24-54, from_goom, irfft2, SiLU gate) and the existing scan seam
 * pallas_scalar_scan(A, X, h0), src/models/pallas_scan.py:341-401. */
int cssm_gated_spectral(const cssm_gated_desc* d, const void* plan, const float* gate_maps,
                        float* xz_planar, void* stream);

/* out_proj from the planar y planes to channels-last y.  cssm.py:584-585. */
int cssm_gated_out_proj(const cssm_gated_desc* d, const cssm_gated_weights* w,
                        const float* xz_planar, float* y, void* stream);

/* Offsets (bytes) of the pieces of the gated workspace, for callers that drive stages. */
typedef struct cssm_gated_ws_layout {
  size_t xz_planar;   /* (B*T, 2C, H, W) float                */
  size_t ctx_sum;     /* (B*T, C) float                       */
  size_t gate_maps;   /* (B*T, H*(W/2+1), 4) float            */
  size_t total;
} cssm_gated_ws_layout;
int cssm_gated_workspace_layout(const cssm_gated_desc* d, cssm_gated_ws_layout* out);

/* -------------------------------------------------------- GatedDeltaNetCSSM --- */
/* Fields of GatedDeltaNetCSSM (cssm.py:4298-4338) read by the general path with
 * gate_type in {factored, dense}, d_k = d_v = delta_key_dim. */
typedef struct cssm_gdn_desc {
  int32_t B, T, H, W, C;
  int32_t delta_key_dim;
  int32_t kernel_size;
  int32_t rope_mode;
  float   rope_base;
  float   spectral_rho;
  int32_t gate_type;
  int32_t short_conv_size;
  int32_t output_norm;            /* 1 = 'rms', 0 = 'none'                            */
  int32_t use_input_gates;
  int32_t output_gate_act;        /* 0 = silu, 1 = sigmoid                            */
  int32_t use_spectral_l2_norm;
  int32_t qkv_conv_size;          /* 1 = Dense only, >1 = depthwise conv first        */
  int32_t no_spectral_clamp;
} cssm_gdn_desc;

/* Parameter tree (cssm.py:4729-5141).  gate order: alpha, beta, B_k, B_v; factored:
 * index 2*g = "<name>_h" (C,H), 2*g+1 = "<name>_w" (C, W/2+1 for alpha/beta, W for
 * B_k/B_v); dense: index g = "<name>". */
typedef struct cssm_gdn_weights {
  const float* kernel;            /* (n_h, ks, ks)                     */
  const float* qkv_dw_kernel;     /* (K,K,1,C) or NULL                 */
  const float* qkv_dw_bias;
  const float* qkv_proj_kernel;   /* (C, 3C)                           */
  const float* qkv_proj_bias;
  const float* conv_t_kernel[3];  /* short_conv_q/k/v (k,1,C) or NULL  */
  const float* conv_t_bias[3];
  const float* gate_kernel[8];
  const float* gate_bias[8];
  const float* gate_proj_kernel;  /* (C, C)                            */
  const float* gate_proj_bias;
  const float* rms_scale;         /* (C) or NULL when output_norm none */
  const float* output_proj_kernel;/* (C, C)                            */
  const float* output_proj_bias;
} cssm_gdn_weights;

size_t cssm_gdn_plan_bytes(const cssm_gdn_desc* d);
size_t cssm_gdn_workspace_bytes(const cssm_gdn_desc* d);

/* Weight-only precompute of W_hat (cssm.py:4713-4734), RoPE tables and the temporal
 * context code (cssm.py:353-383). */
int cssm_gdn_plan_init(const cssm_gdn_desc* d, const cssm_gdn_weights* w,
                       void* plan, size_t plan_bytes, void* stream);

/* Whole block: y = GatedDeltaNetCSSM(x).  Replaces cssm.py:4340-4352, 4685-5141. */
int cssm_gdn_forward(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                     const float* x, float* y, void* workspace, size_t workspace_bytes,
                     void* stream);

/* Last-frame-only variant: y_last (B,H,W,C) = GatedDeltaNetCSSM(x)[:, -1], for callers with a
 * last-frame readout (src/models/simple_cssm.py:482, 524-526).  q/k/v, the gate maps and the state
 * recurrence cover all T steps; the q transforms, the readout, the inverse transforms, gate_proj,
 * RMSNorm and output_proj run for the last frame only.  Same plan and workspace as
 * cssm_gdn_forward. */
int cssm_gdn_forward_last(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                          const float* x, float* y_last, void* workspace,
                          size_t workspace_bytes, void* stream);

/* Static-image fast path (GatedDeltaNetCSSM with static_image_fast_path=True and a 4-D input,
 * src/models/cssm.py:4353-4683): x, y are (B,H,W,C); d->T is num_timesteps.  q, k, v, their
 * spectra and gate_val are computed once per image; alpha_t, beta_t come from the spatial mean of
 * x plus the temporal code; the scan carries M_t, Delta_t and the state rounded to bfloat16 real /
 * imaginary parts with fp32 accumulation (cssm.py:4598-4632) and only the final state is read
 * out.  Requires short_conv_size = 0, use_input_gates = 0, rope_mode none (the reference asserts
 * the same, cssm.py:4354-4370), else CSSM_ERR_UNSUPPORTED.  Plan and workspace: those of
 * cssm_gdn_plan_init / cssm_gdn_workspace_bytes for the same desc. */
int cssm_gdn_forward_static_image(const cssm_gdn_desc* d, const cssm_gdn_weights* w,
                                  const void* plan, const float* x, float* y, void* workspace,
                                  size_t workspace_bytes, void* stream);

/* ================================================================== NoGateCSSM ====
 * The ungated spectral block (src/models/cssm.py:6101-6175): rfft2 of the raw input (no in_proj,
 * no short convs, no RoPE: the reference's __call__ applies none), S_t = K_hat S_{t-1} + X_hat_t
 * in plain complex arithmetic, irfft2, Dense out_proj, minus the input.  x, y: (B,T,H,W,C). */
typedef struct cssm_nogate_desc {
  int32_t B, T, H, W, C;
  int32_t kernel_size;
  float   spectral_rho;     /* 0.999 */
} cssm_nogate_desc;

typedef struct cssm_nogate_weights {
  const float* kernel;           /* (C, ks, ks)   */
  const float* out_proj_kernel;  /* (C, C)        */
  const float* out_proj_bias;    /* (C)           */
} cssm_nogate_weights;

size_t cssm_nogate_plan_bytes(const cssm_nogate_desc* d);
size_t cssm_nogate_workspace_bytes(const cssm_nogate_desc* d);
/* K_hat = squash(rfft2(pad(kernel))) (cssm.py:6127-6147), once per weight set. */
int cssm_nogate_plan_init(const cssm_nogate_desc* d, const cssm_nogate_weights* w, void* plan,
                          size_t plan_bytes, void* stream);
/* y = NoGateCSSM(x) (cssm.py:6124-6175). */
int cssm_nogate_forward(const cssm_nogate_desc* d, const cssm_nogate_weights* w, const void* plan,
                        const float* x, float* y, void* workspace, size_t workspace_bytes,
                        void* stream);

/* ============================================================ AdditiveCSSM (1 state) ====
 * The single-state path of AdditiveCSSM (single_state=True, "add_kqv_1";
 * src/models/cssm.py:2961-3359, 3580-3626): RoPE (optional) -> Dense x_proj -> rfft2 ->
 *   h_t = (d_X,t * K_hat) h_{t-1} + B_X,t * X_hat_t,  h_0 = 0  ->  C_gate,t * h_t -> irfft2 ->
 * Dense output_proj.  The three gates are computed from ctx = mean_{H,W}(rotated x) + temporal
 * code (cssm.py:3127-3131, 353-383): d_X = 0.1 + 0.89 sigmoid(.), B_X = sigmoid(.),
 * C_gate = sigmoid(.), each a per-bin map (H, W/2+1) shared by the channels; gate_type 'dense'
 * (one Dense(H*Wf)) or 'factored' (sigmoid(row + col), cssm.py:3201-3207).  Replaces every
 * scan_mode of that path (associative / ssd / quadratic / pallas, cssm.py:3294-3359): they
 * evaluate the same recurrence.  goom_floor = 1 keeps the 1e-7 magnitude floors of the
 * log-space scan (to_goom, src/models/goom.py:161-173) on K_hat and on B_X * X_hat; 0 is the
 * plain complex recurrence of the other scan modes.  Gates of type conv /
 * dense_decay / dense_io / spectral_conv / low_rank / scalar, learned_init,
 * position_independent_gates and the 2- and 3-state paths are rejected. */
typedef struct cssm_additive_desc {
  int32_t B, T, H, W, C;
  int32_t kernel_size;
  int32_t rope_mode;        /* CSSM_ROPE_* */
  float   rope_base;        /* 10000 */
  float   spectral_rho;     /* 0.999 */
  int32_t gate_type;        /* CSSM_GATE_DENSE, CSSM_GATE_FACTORED or CSSM_GATE_CHANNEL */
  int32_t single_state;     /* must be 1 */
  int32_t goom_floor;       /* 1: scan_mode 'associative' with use_goom; 0: linear scan modes */
} cssm_additive_desc;

typedef struct cssm_additive_weights {
  const float* kernel;              /* (C, ks, ks)                                            */
  const float* x_proj_kernel;       /* (C, C)                                                 */
  const float* x_proj_bias;         /* (C)                                                    */
  /* dense: [0..2] = d_X, B_X, C_gate, kernels (C, H*Wf), biases (H*Wf).
     factored: [0..5] = d_X_h, d_X_w, B_X_h, B_X_w, C_gate_h, C_gate_w, kernels (C,H) / (C,Wf).
     channel (cssm.py:3168-3178): [0] = d_X Dense kernel (C,C); [1], [2] = the 1x1 conv kernels
     (1,1,C,C) of the per-pixel maps B_X (times x_proj before the transform) and C_gate (times the
     output after the inverse transform); biases (C) */
  const float* gate_kernel[6];
  const float* gate_bias[6];
  const float* output_proj_kernel;  /* (C, C)                                                 */
  const float* output_proj_bias;    /* (C)                                                    */
} cssm_additive_weights;

size_t cssm_additive_plan_bytes(const cssm_additive_desc* d);
size_t cssm_additive_workspace_bytes(const cssm_additive_desc* d);
/* K_hat = squash(rfft2(pad(kernel))) (cssm.py:3097-3104), RoPE tables, temporal code. */
int cssm_additive_plan_init(const cssm_additive_desc* d, const cssm_additive_weights* w, void* plan,
                            size_t plan_bytes, void* stream);
/* y = AdditiveCSSM(single_state=True)(x); x, y: (B,T,H,W,C) fp32 channels-last. */
int cssm_additive_forward(const cssm_additive_desc* d, const cssm_additive_weights* w,
                          const void* plan, const float* x, float* y, void* workspace,
                          size_t workspace_bytes, void* stream);

/* ================================================================== DeltaNetCSSM ====
 * The scalar spectral delta rule (src/models/cssm.py:3628-3930): RoPE (optional) -> Dense
 * qkv_proj -> rfft2 of q, k, v per channel; k and v times the spectral input gates B_k, B_v; q
 * and k L2-normalised over the (H, W/2+1) bins of their plane (eps 1e-6 under the root);
 *   A_t = squash(alpha_t W_hat (1 - beta_t |k_t|^2)),  U_t = beta_t v_t conj(k_t),
 *   h_t = A_t h_{t-1} + U_t (h_0 = 0),  o_t = C_gate,t h_t q_t  -> irfft2 -> Dense output_proj.
 * Gates from ctx = mean_{H,W}(rotated x) + temporal code: alpha = 0.1 + 0.89 sigmoid(.), the
 * others sigmoid(.), per-bin maps shared by the channels for gate_type 'dense' or 'factored'
 * (cssm.py:3769-3793).  gate_type 'channel' (the reference's default, cssm.py:3758-3768):
 * alpha, beta are per-channel scalars Dense(C)(ctx); B_k, B_v, C_gate are per-pixel, per-channel
 * maps sigmoid(Conv1x1(C)(rotated x)) applied in the spatial domain (k, v before their
 * transforms, C_gate after the inverse transform).  Replaces every scan_mode of the block
 * (cssm.py:3818-3912); goom_floor as for the additive block (floors on A_t and U_t).
 * gate_type 'scalar', learned_init, position_independent_gates and the bf16 / fp8 split scans
 * are rejected. */
typedef struct cssm_deltanet_desc {
  int32_t B, T, H, W, C;
  int32_t kernel_size;
  int32_t rope_mode;        /* CSSM_ROPE_* */
  float   rope_base;        /* 10000 */
  float   spectral_rho;     /* 0.999 */
  int32_t gate_type;        /* CSSM_GATE_DENSE, CSSM_GATE_FACTORED or CSSM_GATE_CHANNEL */
  int32_t goom_floor;       /* 1: scan_mode 'associative' with use_goom; 0: linear scan modes */
} cssm_deltanet_desc;

typedef struct cssm_deltanet_weights {
  const float* kernel;              /* (C, ks, ks)                                            */
  const float* qkv_proj_kernel;     /* (C, 3C)                                                */
  const float* qkv_proj_bias;       /* (3C)                                                   */
  /* dense: [0..4] = alpha, beta, B_k, B_v, C_gate, kernels (C, H*Wf), biases (H*Wf).
     factored: [0..9] = alpha_h, alpha_w, beta_h, beta_w, B_k_h, B_k_w, B_v_h, B_v_w, C_gate_h,
     C_gate_w, kernels (C,H) / (C,Wf).
     channel: [0..4] = alpha, beta (Dense kernels (C,C)), B_k, B_v, C_gate (Conv kernels
     (1,1,C,C), i.e. (C_in, C_out) row-major), biases (C) */
  const float* gate_kernel[10];
  const float* gate_bias[10];
  const float* output_proj_kernel;  /* (C, C)                                                 */
  const float* output_proj_bias;    /* (C)                                                    */
} cssm_deltanet_weights;

size_t cssm_deltanet_plan_bytes(const cssm_deltanet_desc* d);
size_t cssm_deltanet_workspace_bytes(const cssm_deltanet_desc* d);
/* W_hat = squash(rfft2(pad(kernel))) (cssm.py:3712-3732), RoPE tables, temporal code; with
 * channel gates also the B_k / B_v / C_gate conv kernels packed side by side (weights only). */
int cssm_deltanet_plan_init(const cssm_deltanet_desc* d, const cssm_deltanet_weights* w, void* plan,
                            size_t plan_bytes, void* stream);
/* y = DeltaNetCSSM(x); x, y: (B,T,H,W,C) fp32 channels-last. */
int cssm_deltanet_forward(const cssm_deltanet_desc* d, const cssm_deltanet_weights* w,
                          const void* plan, const float* x, float* y, void* workspace,
                          size_t workspace_bytes, void* stream);

/* ================================================================ SimpleCSSM model ====
 * Inference forward of the reference's SimpleCSSM wrapper around ONE block (depth 1):
 *   stem -> x + block(x) -> last frame -> norm_pre/act -> spatial pool -> norm_post -> head.
 * Replaces SimpleCSSM.__call__ (src/models/simple_cssm.py:173-558) for stem_norm_order 'post',
 * act 'softplus', norm 'layer', frame_readout 'last', pos_embed passed to the block as RoPE
 * (src/models/simple_cssm.py:318-332), no register tokens.  Parameter names: conv{i}/norm{i}
 * (stem layer i = 1..), cssm_0 (the block), norm_pre, norm_post, head. */
typedef struct cssm_simple_desc {
  int32_t B;             /* images or clips                                                   */
  int32_t T;             /* frames per clip; for image input the seq_len the image repeats to */
  int32_t Hin, Win, Cin; /* one input frame (Hin, Win, Cin), channels-last                    */
  int32_t image_input;   /* 1: x is (B,Hin,Win,Cin) (simple_cssm.py:238-241); 0: (B,T,Hin,Win,Cin) */
  int32_t stem_mode;     /* 0 'default': stem_layers x [conv3x3 SAME, softplus, LayerNorm,
                            2x2 max-pool]; 1 'pathtracker': conv1x1, softplus, LayerNorm       */
  int32_t stem_layers;   /* 1..4 for the default stem                                         */
  int32_t embed_dim;     /* multiple of 4, <= 64                                              */
  int32_t block;         /* 0 GatedCSSM (block_desc is a cssm_gated_desc), 1 GatedDeltaNetCSSM,
                            2 NoGateCSSM, 3 AdditiveCSSM single-state, 4 DeltaNetCSSM (their own
                            descriptors; these three ignore CSSM_SIMPLE_LAST_FRAME_ONLY)       */
  int32_t pool_type;     /* 0 mean, 1 max                                                     */
  int32_t readout_norm;  /* 0 'pre' (norm -> act), 1 'post' (act -> norm)                     */
  int32_t num_classes;   /* 1..64                                                             */
} cssm_simple_desc;

typedef struct cssm_simple_weights {
  const float* conv_kernel[4];   /* stem conv i: (k,k,cin_i,embed_dim), k = 3 (default) or 1   */
  const float* conv_bias[4];     /* (embed_dim)                                                */
  const float* norm_scale[4];    /* stem LayerNorm i                                           */
  const float* norm_bias[4];
  const float* norm_pre_scale;   /* (embed_dim)                                                */
  const float* norm_pre_bias;
  const float* norm_post_scale;
  const float* norm_post_bias;
  const float* head_kernel;      /* (embed_dim, num_classes)                                   */
  const float* head_bias;        /* (num_classes)                                              */
} cssm_simple_weights;

/* flags of cssm_simple_forward* */
#define CSSM_SIMPLE_LAST_FRAME_ONLY 1   /* evaluate the block through its last-frame-only entry
                                           point (same logits; the earlier output frames, which
                                           the readout never reads, are not produced) */

/* block_desc: the cssm_gated_desc / cssm_gdn_desc of the block; its B, T, H, W, C must equal the
 * stem's output (B, T, Hin >> stem_layers rounded up, ..., embed_dim).  0 if inconsistent. */
size_t cssm_simple_workspace_bytes(const cssm_simple_desc* d, const void* block_desc);

/* Stem alone: x frames -> features.  Image input: feat is (B,H,W,C) (the frame that the block
 * then reads for every t); clip input: (B,T,H,W,C).  Replaces simple_cssm.py:244-281. */
int cssm_simple_stem(const cssm_simple_desc* d, const cssm_simple_weights* w, const float* x,
                     float* feat, void* workspace, size_t workspace_bytes, void* stream);

/* Readout alone: logits (B,num_classes) from the block's last output frame y_last (B,H,W,C)
 * plus the residual frame res (B,H,W,C) (simple_cssm.py:482, 523-556).  y_stride / res_stride:
 * floats between consecutive batch elements of each (H*W*C when packed).  partial: scratch of
 * B * ceil(H/8) * C floats. */
int cssm_simple_readout(const cssm_simple_desc* d, const cssm_simple_weights* w, int32_t H,
                        int32_t W, const float* y_last, size_t y_stride, const float* res,
                        size_t res_stride, float* partial, float* logits, void* stream);

/* Whole model on device buffers: x as described by image_input, logits (B, num_classes). */
int cssm_simple_forward(const cssm_simple_desc* d, const cssm_simple_weights* w,
                        const void* block_desc, const void* block_weights, const void* block_plan,
                        const float* x, float* logits, void* workspace, size_t workspace_bytes,
                        int32_t flags, void* stream);

/* Same with x and logits in HOST memory (pinned for full copy speed): copies x to the device
 * (staging area inside the workspace: cssm_simple_host_workspace_bytes), runs the model, copies
 * the logits back and waits for the stream. */
size_t cssm_simple_host_workspace_bytes(const cssm_simple_desc* d, const void* block_desc);
int cssm_simple_forward_host(const cssm_simple_desc* d, const cssm_simple_weights* w,
                             const void* block_desc, const void* block_weights,
                             const void* block_plan, const float* x_host, float* logits_host,
                             void* workspace, size_t workspace_bytes, int32_t flags, void* stream);

/* ------------------------------------------------------------ CSSM-SHViT (bf16) --- */
/* Inference forward of the CSSM-SHViT image classifier around gated mixers (src/models/
 * cssm_shvit.py:269-460 with the layers of src/models/shvit.py:34-262), as the reference runs it
 * with dtype = bfloat16: activations are bfloat16 channels-last, parameters float32 in the
 * reference's layout (Dense (in, out), conv HWIO, BatchNorm scale / bias / running mean / var),
 * accumulation float32, logits float32.  Image input only (the model repeats it over
 * num_timesteps), cssm_type 'gated', block_norm 'global_layer', inference (deterministic) mode.
 * The Dense layers and the 3x3 stride-2 ConvBN layers run as bf16 tcgen05 GEMMs (the convs as
 * implicit GEMMs), BatchNorm folded into the weights. */
#define CSSM_SHVIT_MAX_BLOCKS 16

/* One block of a stage.  is_cssm = 0: ConvBlock (shvit.py:219-262); 1: CSSMSHViTBlock with a
 * GatedCSSM mixer (cssm_shvit.py:19-266). */
typedef struct cssm_shvit_block_desc {
  int32_t B, H, W, C;               /* block input (B,H,W,C)                              */
  int32_t is_cssm;
  int32_t hidden;                   /* int(dim * mlp_ratio)                               */
  int32_t num_timesteps;            /* T of the mixer                                     */
  int32_t kernel_size;              /* spectral kernel of the mixer                       */
  int32_t use_pos_conv, use_dwconv;
  int32_t rope_mode; float rope_base; float spectral_rho;
  int32_t gate_activation, short_conv_size, short_conv_spatial_size, gate_type;
} cssm_shvit_block_desc;

typedef struct cssm_shvit_block_weights {
  const float* norm1_scale; const float* norm1_bias;     /* (C)                           */
  const float* norm2_scale; const float* norm2_bias;
  const float* dw_kernel; const float* dw_bias;          /* ConvBlock dwconv (7,7,1,C); CSSM block pos_conv (3,3,1,C) or NULL */
  const float* pw_kernel; const float* pw_bias;          /* ConvBlock pwconv (C,C)        */
  const float* fc1_kernel; const float* fc1_bias;        /* (C,hidden)                    */
  const float* fc2_kernel; const float* fc2_bias;        /* (hidden,C)                    */
  const float* mlp_dw_kernel; const float* mlp_dw_bias;  /* CSSM block Mlp dwconv (3,3,1,hidden) or NULL */
  cssm_gated_weights cssm;                               /* CSSM block: the mixer         */
} cssm_shvit_block_weights;

typedef struct cssm_shvit_convbn {       /* ConvBN, shvit.py:34-61 */
  const float* kernel;                   /* (3,3,Cin,Cout), no bias */
  const float* bn_scale; const float* bn_bias; const float* bn_mean; const float* bn_var;
} cssm_shvit_convbn;

typedef struct cssm_shvit_desc {
  int32_t B, H, W, Cin;             /* images (B,H,W,Cin) bfloat16                         */
  int32_t embed_dims[4], depths[4], use_cssm[4], kernel_sizes[4];
  int32_t num_classes, num_timesteps;
  float   mlp_ratio;
  int32_t use_pos_conv, use_dwconv;
  int32_t head_pool;                /* 0 max, 1 mean (cssm_shvit.py:436-439)               */
  int32_t rope_mode; float rope_base; float spectral_rho;
  int32_t gate_activation, short_conv_size, short_conv_spatial_size, gate_type;
} cssm_shvit_desc;

typedef struct cssm_shvit_weights {
  cssm_shvit_convbn patch[2];                            /* patch_embed/ConvBN_0, ConvBN_1 */
  cssm_shvit_convbn down[3];                             /* downsample1..3/ConvBN_0        */
  cssm_shvit_block_weights blocks[CSSM_SHVIT_MAX_BLOCKS]; /* stage0_block0, ... in order   */
  const float* norm_scale; const float* norm_bias;       /* final LayerNorm                */
  const float* head_kernel; const float* head_bias;      /* (C3, num_classes)              */
} cssm_shvit_weights;

/* One block on device buffers: x, y (B,H,W,C) bfloat16.  Replaces ConvBlock.__call__
 * (shvit.py:232-262) / CSSMSHViTBlock.__call__ for a 4-D input (cssm_shvit.py:66-266). */
size_t cssm_shvit_block_plan_bytes(const cssm_shvit_block_desc* d);
size_t cssm_shvit_block_workspace_bytes(const cssm_shvit_block_desc* d);
int cssm_shvit_block_plan_init(const cssm_shvit_block_desc* d, const cssm_shvit_block_weights* w,
                               void* plan, size_t plan_bytes, void* stream);
int cssm_shvit_block_forward(const cssm_shvit_block_desc* d, const cssm_shvit_block_weights* w,
                             const void* plan, const void* x_bf16, void* y_bf16, void* workspace,
                             size_t workspace_bytes, void* stream);

/* Whole model: logits (B, num_classes) float32 = CSSMSHViT(x, training=False)
 * (cssm_shvit.py:324-460).  The plan holds the packed bf16 weights (call plan_init again when the
 * parameters change). */
size_t cssm_shvit_plan_bytes(const cssm_shvit_desc* d);
size_t cssm_shvit_workspace_bytes(const cssm_shvit_desc* d);
int cssm_shvit_plan_init(const cssm_shvit_desc* d, const cssm_shvit_weights* w, void* plan,
                         size_t plan_bytes, void* stream);
int cssm_shvit_forward(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                       const void* x_bf16, float* logits, void* workspace, size_t workspace_bytes,
                       void* stream);
/* cssm_shvit_forward with a launch trace (no counterpart in the reference): before every kernel of
 * the forward an event of `events` (cudaEvent_t created by the caller, timing enabled) is recorded
 * on `stream`, and the kernel kind and the algorithmic bytes of that launch (inputs + outputs +
 * weights) are written beside it; one more entry (CSSM_SHVIT_K_END) marks the end.  `count` returns
 * the number of entries used.  Nothing is kept after the call returns. */
enum {
  CSSM_SHVIT_K_STEM_CONV = 0, CSSM_SHVIT_K_CONV_GEMM = 1, CSSM_SHVIT_K_GEMM = 2,
  CSSM_SHVIT_K_LAYERNORM = 3, CSSM_SHVIT_K_DWCONV7 = 4, CSSM_SHVIT_K_DWCONV3 = 5,
  CSSM_SHVIT_K_SAMPLE_NORM = 6, CSSM_SHVIT_K_PLANE_SUM = 7, CSSM_SHVIT_K_GATES = 8,
  CSSM_SHVIT_K_SPECTRAL = 9, CSSM_SHVIT_K_POOL = 10, CSSM_SHVIT_K_HEAD = 11,
  CSSM_SHVIT_K_MIXER_F32 = 12, CSSM_SHVIT_K_ADD_RES = 13, CSSM_SHVIT_K_MLP = 14, CSSM_SHVIT_K_END = 15
};
typedef struct cssm_shvit_trace {
  void** events; int32_t* kinds; double* bytes;
  int32_t capacity; int32_t count;
} cssm_shvit_trace;
int cssm_shvit_forward_timed(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                             const void* x_bf16, float* logits, void* workspace, size_t workspace_bytes,
                             void* stream, cssm_shvit_trace* trace);

/* Same with the images and the logits in HOST memory (pinned for full copy speed).  The batch is
 * cut into up to four chunks whose host->device copies run on an internal stream while the previous
 * chunk computes (two staging buffers inside the workspace, ordered by events); the logits of all
 * chunks return in one copy and the call waits for it.  The internal stream and events live for
 * the duration of the call only. */
size_t cssm_shvit_host_workspace_bytes(const cssm_shvit_desc* d);
int cssm_shvit_forward_host(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                            const void* x_bf16_host, float* logits_host, void* workspace,
                            size_t workspace_bytes, void* stream);

/* Streaming form of the host entry point, for a loop that feeds batch after batch (the reference's
 * evaluation loop, main.py:522-561, prefetches its next batch the same way): while batch i computes,
 * the images of batch i+1 are copied to the device on the pipe's own stream.
 *   cssm_host_pipe_create / _destroy: a caller-owned handle holding one copy stream, two
 *     events and the address of the prefetched batch; it owns no device memory.
 *   cssm_shvit_forward_host_pipelined(..., x_bf16_host, x_next_bf16_host, ...): computes the logits of
 *     x_bf16_host for the whole batch at once and returns after they have arrived on the host.  If the
 *     previous call on this pipe named the same address as its x_next, the images are already on the
 *     device (or still arriving: the compute stream waits for the copy's event); otherwise they are
 *     copied first.  x_next_bf16_host (may be NULL) starts copying into the other input buffer before
 *     the call computes; the caller must leave that host buffer unchanged until the next call on this
 *     pipe or its destruction.  Workspace: cssm_shvit_host_pipe_workspace_bytes (the model workspace,
 *     two whole-batch input buffers, the logits). */
typedef struct cssm_host_pipe cssm_host_pipe;
int cssm_host_pipe_create(cssm_host_pipe** pipe);
int cssm_host_pipe_destroy(cssm_host_pipe* pipe);
size_t cssm_shvit_host_pipe_workspace_bytes(const cssm_shvit_desc* d);
int cssm_shvit_forward_host_pipelined(const cssm_shvit_desc* d, const cssm_shvit_weights* w, const void* plan,
                                      cssm_host_pipe* pipe, const void* x_bf16_host,
                                      const void* x_next_bf16_host, float* logits_host, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* The streaming form for the SimpleCSSM models (float32 images or clips): same pipe handle, same
 * contract as cssm_shvit_forward_host_pipelined, arguments of cssm_simple_forward_host. */
size_t cssm_simple_host_pipe_workspace_bytes(const cssm_simple_desc* d, const void* block_desc);
int cssm_simple_forward_host_pipelined(const cssm_simple_desc* d, const cssm_simple_weights* w,
                                       const void* block_desc, const void* block_weights,
                                       const void* block_plan, cssm_host_pipe* pipe, const float* x_host,
                                       const float* x_next_host, float* logits_host, void* workspace,
                                       size_t workspace_bytes, int32_t flags, void* stream);

/* The bf16 tensor-core GEMM of the model's Dense layers on its own (nn.Dense with dtype bfloat16:
 * shvit.py:165-180; cssm.py:481, 584 inside a bf16 model):
 *   out (M,N) bf16 = act(A (M,K) bf16 @ kernel (K,N) + bias) [+ res (M,N) bf16]
 * `wt` is the kernel packed by cssm_bf16_pack_weight: (N, ldw) bf16, ldw = cssm_bf16_packed_ld(K).
 * act: 0 none, 1 gelu (tanh form, jax.nn.gelu's default), 2 silu.  K and N multiples of 32. */
int32_t cssm_bf16_packed_ld(int32_t K);
int cssm_bf16_pack_weight(const float* kernel, int32_t K, int32_t N, const float* col_scale,
                          void* wt, void* stream);
int cssm_bf16_gemm(const void* A, int32_t M, int32_t K, const void* wt, int32_t N, const float* bias,
                   int32_t act, const void* res, void* out, void* stream);
/* The whole Mlp of a block (shvit.py:165-180: fc1 C -> Hd, gelu, fc2 Hd -> C) plus the block's residual
 * in one kernel, the hidden tensor staying on the SM:
 *   out (M,C) bf16 = res (M,C) bf16 + gelu(a (M,C) bf16 @ W1 + b1) @ W2 + b2
 * w1t / w2t are W1 (C,Hd) / W2 (Hd,C) packed by cssm_bf16_pack_weight.  Built for C = 64, Hd = 256 (the
 * stage-0 ConvBlock of CSSM-SHViT s1); other sizes return CSSM_ERR_UNSUPPORTED and the caller runs two
 * cssm_bf16_gemm calls instead, as the model's forward pass does. */
int cssm_bf16_mlp(const void* a, int32_t M, int32_t C, int32_t Hd, const void* w1t, const float* b1,
                  const void* w2t, const float* b2, const void* res, void* out, void* stream);
/* 3x3 stride-2 'SAME' convolution (nn.Conv inside ConvBN, shvit.py:45-54) as an implicit GEMM:
 * x (B,Hi,Wi,Cin) bf16 -> out (B,ceil(Hi/2),ceil(Wi/2),Cout) bf16; `wt` = the HWIO kernel (3,3,Cin,Cout)
 * packed by cssm_bf16_pack_conv3x3s2_weight into (Cout, cssm_bf16_conv3x3s2_packed_ld(Cin, Wi, Cout)) bf16
 * (col_scale = the BatchNorm factor; the layout depends on Cin, Cout and the parity of the input width). */
int32_t cssm_bf16_conv3x3s2_packed_ld(int32_t Cin, int32_t Wi, int32_t Cout);
int cssm_bf16_pack_conv3x3s2_weight(const float* kernel, int32_t Cin, int32_t Cout, int32_t Wi,
                                    const float* col_scale, void* wt, void* stream);
int cssm_bf16_conv3x3s2(const void* x, int32_t B, int32_t Hi, int32_t Wi, int32_t Cin, const void* wt,
                        int32_t Cout, const float* bias, int32_t act, void* out, void* stream);

/* ---- device-side error word (no counterpart in the reference) ----
 * Kernels of this library wait on hardware barriers (TMA copies landing, tensor-core tiles
 * finishing) with an iteration limit.  A wait that runs out does not hang or trap: the CTA records
 * a code in a device word, stops storing results and winds down, and the forward call that
 * launched it has long since returned CSSM_OK (calls are asynchronous).  After synchronising the
 * stream, cssm_device_error copies that word to *out: 0 = no wait ever expired on the current
 * device since the last clear; low byte = fp32 tensor-core projection kernels (1 producer, 2 MMA
 * issuer, 3 drain, 4 epilogue), next byte = fused spectral kernels (1 input plane, 2 z plane),
 * third byte = bf16 tensor-core GEMM (5 TMA producer, 6 MMA issuer, 7 drain, 8 epilogue, 9 im2col
 * producer), top byte = fused Mlp kernel (1 TMA producer, 2-6 MMA issuers, 8 drain, 9-13 epilogue).
 * A non-zero value means the outputs of the calls since the last clear are not to be trusted.
 * clear != 0 resets the word after reading it.  The call copies from the device on the legacy
 * default stream (it waits for work on blocking streams). */
int cssm_device_error(int* out, int clear);

/* cssm_gdn_forward with per-stage timing: `stage_events` is an array of 8 cudaEvent_t created by
 * the caller; events[i] is recorded on `stream` before stage i (0 dwconv+ctx, 1 qkv_proj,
 * 2 gate_proj, 3 gates, 4 short convs, 5 fused spectral kernel, 6 norm+gate+output_proj) and
 * events[7] at the end.  Nothing is kept after the call returns. */
int cssm_gdn_forward_timed(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                           const float* x, float* y, void* workspace, size_t workspace_bytes,
                           void* stream, void** stage_events);

/* ---- entry point that allocates nothing (no counterpart in the reference) ----
 * The reference has nothing like this: it is for hosts that may not call cudaMalloc at all
 * (a plugin running inside another framework's step, whose allocator owns the device memory;
 * a sandboxed or latency-bound service that is only permitted to launch work).  It is
 * cssm_gated_forward with the block's scratch memory taken from one fixed array inside the
 * library image instead of a caller workspace.  The caller still passes plan, x and y.
 *  - Limit: cssm_gated_workspace_bytes(d) must be <= cssm_static_scratch_bytes() (64 MiB);
 *    larger problems return CSSM_ERR_SIZE_LIMIT.  Every GPU that loads the library carries
 *    the 64 MiB array until the process exits.
 *  - The first call on each device looks up the array's device address (with that device
 *    current) and keeps it for the life of the process; make that first call before starting
 *    any stream capture.  The address dies with the device's primary context: do not call
 *    this entry point again after cudaDeviceReset.
 *  - All calls on a device share the array: two calls whose kernels overlap on the GPU
 *    (different streams) race.  Nothing needs clearing between calls: each part of the
 *    scratch is rewritten before it is read.
 *  - Calls no cudaMalloc / cudaFree or any allocating routine. */
size_t cssm_static_scratch_bytes(void);
int cssm_gated_forward_static(const cssm_gated_desc* d, const cssm_gated_weights* w,
                              const void* plan, const float* x, float* y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CSSM_B200_H_ */
