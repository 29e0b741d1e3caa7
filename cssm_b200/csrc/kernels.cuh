// Argument structs and host launchers of the kernels, shared by the kernel sources and the
// C-ABI sources.
#pragma once
#include "common.cuh"

namespace cssm {

int launch_khat(const float* k, cf* out, int nch, int ks, int H, int W, float rho, int squash,
                int floor_eps, int path, cudaStream_t st);
int launch_rope_tables(float2* tt, float2* th, float2* tw, int T, int H, int W, int C, int mode,
                       float base, cudaStream_t st);
int launch_tcode(float* out, int T, int C, float base, cudaStream_t st);

struct StencilArgs {
  float* buf; int planes_per_frame, plane0;   // plane (frame*planes_per_frame + plane0 + c)
  int B, T, C, H, W;
  const float* wsp; const float* bsp; int ksp;   // (k,k,1,C), (C)
  const float* wt; const float* bt; int kt;      // (k,1,C), (C)
  int act;
  const float* post;                             // (B*T, H*W) or nullptr
  float* sums;                                   // (B*T, C) or nullptr
};
int launch_plane_stencil(const StencilArgs& s, cudaStream_t st);

struct GatedGateArgs {
  const float* ctx_sum; int BT, C, H, W, gate_type, act, path;
  const float* gk[6]; const float* gb[6];
  float4* maps;
};
int launch_gated_gates(const GatedGateArgs& g, cudaStream_t st);

int launch_gated_spectral(const cssm_gated_desc& d, const cf* khat, const float* gates,
                          float* xz, cudaStream_t st);
size_t generic_smem_bytes(int H, int W);

}  // namespace cssm
