// Argument structs and host launchers of the kernels, shared by the kernel sources and the
// C-ABI sources.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

namespace cssm {

int launch_khat(const float* k, cf* out, int nch, int ks, int H, int W, float rho, int squash,
                int floor_eps, int path, cudaStream_t st);
int launch_rope_tables(float2* tt, float2* th, float2* tw, float* nz, int T, int H, int W, int C,
                       int mode, float base, cudaStream_t st);
int launch_tcode(float* out, int T, int C, float base, cudaStream_t st);

struct StencilArgs {
  float* buf; int planes_per_frame, plane0;   // plane (frame*planes_per_frame + plane0 + c)
  int B, T, C, H, W;
  const float* wsp; const float* bsp; int ksp;   // (k,k,1,C), (C)
  const float* wt; const float* bt; int kt;      // (k,1,C), (C)
  int act;
  const float* post;                             // per-pixel factor or nullptr:
  int post_stride, post_off;                     //   post[(frame*H*W + px)*post_stride + post_off]
  float* sums;                                   // (B*T, C) or nullptr
};
int launch_plane_stencil(const StencilArgs& s, cudaStream_t st);

// temporal conv + SiLU (+ input gates) on the q, k, v planes of the GDN block in one launch
struct QkvTconvArgs {
  float* buf;                     // planar (B*T, 3C, H*W), in place
  int B, T, C, HW, kt;
  const float* wt[3]; const float* bt[3];   // short_conv_q/k/v: (kt,1,C), (C)
  const float2* bkv;              // (B*T, H*W) {B_k, B_v} or nullptr (no input gates)
};
int launch_qkv_temporal_conv(const QkvTconvArgs& a, cudaStream_t st);   // CSSM_ERR_UNSUPPORTED: use the plane stencil

struct GatedGateArgs {
  const float* ctx_sum; int BT, C, H, W, gate_type, act, path;
  const float* gk[6]; const float* gb[6];
  float4* maps;
};
int launch_gated_gates(const GatedGateArgs& g, cudaStream_t st);

// last_only != 0: only the last step's output plane is produced (inverse transforms, the z
// plane and the stores of earlier steps are skipped; the recurrence still runs over all T)
int launch_gated_spectral(const cssm_gated_desc& d, const cf* khat, const float* gates,
                          float* xz, int last_only, cudaStream_t st);
// nogate == 1: the ungated recurrence S_t = K_hat S_{t-1} + X_hat_t (NoGateCSSM): `gates` is not
// read and the z planes of the (B*T, 2C, H, W) buffer are neither read nor written.
// nogate == 2: gate maps as in the gated block, but no z planes (single-state AdditiveCSSM)
int launch_spectral(int B, int T, int H, int W, int C, const cf* khat, const float* gates,
                    float* xz, int last_only, int nogate, cudaStream_t st, const float* dchan = nullptr);
size_t generic_smem_bytes(int H, int W);
int read_spec_error(int* out, int clear);

// ---- DeltaNet block (scalar delta rule) ----
struct DnSpectralArgs {
  float* qkv;               // planar (BT, 3C, H, W): q, k, v; the output overwrites the v planes
  const cf* what;           // (C, H*Wf) squashed kernel spectrum, bins at bin_index(path, ...)
  const float4* abkv;       // (BT, H*Wf) {alpha, beta, B_k, B_v}, same bin order
  const float* cg;          // (BT, H*Wf) C_gate / (H*W)
  const float2* chan;       // channel gates: (BT, C) {alpha, beta}; then abkv and cg are not read
                            // (B_k = B_v = 1, output scale 1/(H*W)); nullptr = per-bin maps
  int B, T, C, H, W;
  float rho;
  int goom_floor;
};
int launch_deltanet_spectral_r64(const DnSpectralArgs& a, cudaStream_t st);
int launch_deltanet_spectral_r32(const DnSpectralArgs& a, cudaStream_t st);

// ---- GDN block ----
struct GdnDwArgs {
  const float* x; float* out;            // channels-last (BT, H, W, C); out may be nullptr
  const float* wk; const float* bias;    // (K,K,1,C), (C)
  int ksz;                               // <= 1: no conv (only the context sums)
  int BT, T, H, W, C;
  int x_bcast;                           // 1: x holds one frame per clip (frame fr reads fr / T)
  const float2* rope_t; const float2* rope_h; const float2* rope_w;   // nullptr = no RoPE
  float* ctx_part;                       // (BT, H, C) row sums of the rotated input
};
int launch_rope_dwconv_cl(const GdnDwArgs& a, cudaStream_t st);

struct GdnGateArgs {
  const float* ctx_part; const float* tcode;   // (BT,H,C), (T,C)
  int BT, T, C, H, W, gate_type, use_input_gates, path;
  int ctx_per_clip;                      // 1: ctx_part holds one frame per clip (frame fr reads fr / T)
  const float* gk[8]; const float* gb[8];
  int nh;                                // heads (channel gates: one {alpha, beta} map per head)
  float2* ab;                            // (BT, H*Wf) {alpha, beta} in spectral bin order; channel gates: (BT, nh, H*Wf)
  float2* bkv;                           // (BT, H*W)  {B_k, B_v} (not written for channel gates)
};
int launch_gdn_gates(const GdnGateArgs& g, cudaStream_t st);

struct GdnSpectralArgs {
  float* qkv;                // planar (BT, 3C, H, W): q planes, k planes, v planes (o overwrites v)
  const cf* what;            // (n_h, H*Wf) in spectral bin order
  const float2* ab;          // (BT, ab_heads, H*Wf)
  int ab_heads;              // 1: one gate map per frame; C/dk: one per (frame, head)
  cf* state;                 // (B*n_h, dk, dk, H*Wf) scratch for the matrix state
  int B, T, C, H, W, dk, use_l2;
  int static_image;          // != 0: static-image fast path: qkv holds ONE frame per batch element
                             // (B, 3C, H, W); ab holds the gates of T steps; the whole scan runs per
                             // bin with a bf16 carry and only the final readout is produced
  int last_only;             // != 0: only the last step's output planes are produced (the q
                             // transforms, readout and inverse transforms of earlier steps are skipped)
};
int launch_gdn_spectral(const GdnSpectralArgs& a, cudaStream_t st);
size_t gdn_generic_smem_bytes(int H, int W, int dk);

// ---- bf16 tensor-core GEMM with a K loop (csrc/gemm_bf16.cu) ----
struct Bf16GemmArgs {
  // plain mode (ksz == 0): A is (M, K) bf16 row-major with row stride lda.
  // conv mode (ksz > 0): A is a channels-last image batch (Bimg, Hi, Wi, Cin) and row m is output
  //   pixel (b, ho, wo); K = ksz*ksz*Cin in (tap row, tap column, channel) order; zero padding of
  //   pad_h / pad_w pixels before the first row / column (whatever falls outside the image is 0).
  const __nv_bfloat16* A;
  int M, N, K, lda;
  int ksz, stride, Hi, Wi, Cin, Ho, Wo, pad_h, pad_w;
  const __nv_bfloat16* Wt;   // (N, ldw) bf16: weights transposed to K-major, ldw >= round_up(K, 64), zero padded
  int ldw;
  const float* bias;         // (N) or nullptr
  int act;                   // 0 none, 1 gelu (tanh form), 2 silu
  const __nv_bfloat16* res;  // (M, ldr) added after the activation, or nullptr
  int ldr;
  __nv_bfloat16* out;        // (M, ldo) bf16
  float* out_f32;            // reserved (must be nullptr)
  int ldo;
  int Kpad, BN, stages;      // filled in by the launcher
  int nacc, ostg;            // TMEM accumulators; staging slots per epilogue half (launcher)
  int wres;                  // 1: the weights stay resident in shared memory (launcher)
  // conv mode through TMA (filled in by the launcher): an M tile is a patch of Bbox images x Hbox
  // output rows x Wbox output columns (at most 128 pixels); K block kb is `kb_ch` channels from
  // channel (kb % kb_per_tap) * kb_ch of window position kb / kb_per_tap (row = pos / pos_w,
  // column = pos % pos_w, in units of w_unit input pixels).
  int conv_tma, Wbox, Hbox, Bbox, tiles_w, tiles_h, kb_per_tap, pos_w, Bimg;
};
int launch_gemm_bf16(Bf16GemmArgs g, cudaStream_t st);
// Weight layout of the 3x3 stride-2 conv for an input of Cin channels and width Wi: 0 = the HWIO
// kernel flattened to (9*Cin, Cout) (K = (row, column, channel)); 1 = the wide-pixel layout for
// Cin = 32, even Wi and Cout a multiple of 64: per kernel row two K blocks of 64 = [column 0 | column 1] and
// [column 2 | zeros], so that every K block is one 128-byte pair of adjacent input pixels.
int conv3x3s2_weight_layout(int Cin, int Wi, int Cout);
int conv3x3s2_packed_k(int Cin, int Wi, int Cout);
int gemm_bf16_pick_bn(int N);
int read_bf16_error(int* out, int clear);

// fused fc1 + GELU + fc2 + residual of the 64-channel ConvBlock (csrc/mlp_fused.cu)
bool mlp_fused_supported(int C, int Hd);
int launch_mlp_fused(const __nv_bfloat16* a, int M, const __nv_bfloat16* w1t, int ld1, const float* b1,
                     const __nv_bfloat16* w2t, int ld2, const float* b2, const __nv_bfloat16* res,
                     __nv_bfloat16* out, cudaStream_t st);
int read_mlp_error(int* out, int clear);

// ---- bf16 model kernels (csrc/shvit_kernels.cu, csrc/spectral_cl.cu) ----
int launch_pack_wt(const float* src, int K, int N, const float* colscale, __nv_bfloat16* dst, int ldw,
                   cudaStream_t st);
int launch_pack_conv3x3(const float* src, int Cin, int N, int Wi, const float* colscale, __nv_bfloat16* dst,
                        cudaStream_t st);
int launch_bn_fold(const float* scale, const float* bias, const float* mean, const float* var, int C,
                   float* oscale, float* obias, cudaStream_t st);
int launch_affine_vec(const float* a, const float* s, const float* b, int C, float* out, cudaStream_t st);
int launch_fill(float* p, int n, float v, cudaStream_t st);
int launch_scale_cols(const float* src, int K, int N, const float* s, float* out, cudaStream_t st);
int launch_stem_conv1(const __nv_bfloat16* x, const float* wk, const float* bias, __nv_bfloat16* y,
                      int Nimg, int Hi, int Wi, int Cin, int Co, int gelu, cudaStream_t st);
// wk == nullptr: no taps (only the pre-affine / centre term)
int launch_dwconv_cl(const __nv_bfloat16* x, const float* wk, const float* bias, const float* pre_a,
                     const float* pre_b, __nv_bfloat16* y, float* y_f32, int Nimg, int H, int W, int C,
                     int ks, int add_centre, int gelu, cudaStream_t st);
int launch_layernorm_cl(const __nv_bfloat16* x, const float* scale, const float* bias, __nv_bfloat16* y,
                        long long npix, int C, cudaStream_t st);
int launch_sample_norm(const __nv_bfloat16* x, const float* scale, const float* bias, float* a, float* b,
                       int Nimg, int per, int C, cudaStream_t st);
int launch_plane_sum_cl(const __nv_bfloat16* x, int ld, int Nimg, int P, int C, float* sums, cudaStream_t st);
int launch_pool_cl(const __nv_bfloat16* x, int Nimg, int P, int C, int use_max, float* pooled, cudaStream_t st);
int launch_head(const float* pooled, const float* W, const float* b, float* logits, int Nimg, int C, int K,
                cudaStream_t st);
int launch_f32_to_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t st);
int launch_add_res(const __nv_bfloat16* res, const float* yv, __nv_bfloat16* out, long long n, cudaStream_t st);
bool spectral_cl_supported(int H, int W, int C, int T);
int launch_gated_spectral_cl(const __nv_bfloat16* xz, int ld, int Nimg, int H, int W, int C,
                             const float* gates, __nv_bfloat16* y, int ldy, cudaStream_t st);

// ---- whole-block drivers shared by the C-ABI sources ----
// last_only: y is (B,H,W,C), the last output frame.  x_bcast: x is (B,H,W,C), one frame per
// batch element standing for all T frames (an image repeated over the sequence).
int gated_forward_internal(const cssm_gated_desc* d, const cssm_gated_weights* w, const void* plan,
                           const float* x, float* y, void* workspace, size_t workspace_bytes,
                           void* stream, int last_only, int x_bcast);
int gdn_forward_internal(const cssm_gdn_desc* d, const cssm_gdn_weights* w, const void* plan,
                         const float* x, float* y, void* workspace, size_t workspace_bytes,
                         void* stream, int last_only, int x_bcast);

}  // namespace cssm
