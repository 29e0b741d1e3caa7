// extern "C" entry points of the ungated spectral block (NoGateCSSM): rfft2 of the raw input,
// S_t = K_hat S_{t-1} + X_hat_t, irfft2, out_proj, minus the input (src/models/cssm.py:6101-6175).
#include <string.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"

namespace cssm {

// channels-last (frames, HW, C) -> x_main planes of the planar (frames, 2C, HW) buffer that the
// spectral kernels work on (the z planes stay untouched).  32 pixels x 32 channels per tile.
__global__ void __launch_bounds__(256) cl_to_planar_kernel(const float* __restrict__ x,
                                                           float* __restrict__ planar, int frames,
                                                           int HW, int C) {
  __shared__ float tile[32][33];
  const int ptiles = (HW + 31) / 32, ctiles = (C + 31) / 32;
  int bid = blockIdx.x;
  const int ct = bid % ctiles; bid /= ctiles;
  const int pt = bid % ptiles;
  const int fr = bid / ptiles;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int px = pt * 32 + ty + 8 * r, c = ct * 32 + tx;
    tile[ty + 8 * r][tx] = (px < HW && c < C) ? x[((size_t)fr * HW + px) * C + c] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int c = ct * 32 + ty + 8 * r, px = pt * 32 + tx;
    if (px < HW && c < C) planar[((size_t)fr * 2 * C + c) * HW + px] = tile[tx][ty + 8 * r];
  }
}

static int nogate_validate(const cssm_nogate_desc* d) {
  if (!d) return CSSM_ERR_NULL;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->W <= 0 || d->C <= 0 || d->kernel_size <= 0)
    return CSSM_ERR_DIMS;
  if (d->C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  const bool crop_h = d->kernel_size > d->H, crop_w = d->kernel_size > d->W;
  if (crop_h != crop_w) return CSSM_ERR_UNSUPPORTED;
  if (spectral_path(d->H, d->W) == PATH_GENERIC && generic_smem_bytes(d->H, d->W) > 200 * 1024)
    return CSSM_ERR_UNSUPPORTED;
  return CSSM_OK;
}

static size_t nogate_khat_bytes(const cssm_nogate_desc& d) {
  return round_up((size_t)d.C * d.H * (d.W / 2 + 1) * sizeof(cf), 256);
}

}  // namespace cssm

using namespace cssm;

extern "C" {

size_t cssm_nogate_plan_bytes(const cssm_nogate_desc* d) {
  return nogate_validate(d) == CSSM_OK ? nogate_khat_bytes(*d) : 0;
}

size_t cssm_nogate_workspace_bytes(const cssm_nogate_desc* d) {
  if (nogate_validate(d) != CSSM_OK) return 0;
  return round_up((size_t)d->B * d->T * 2 * d->C * d->H * d->W * sizeof(float), 256);
}

int cssm_nogate_plan_init(const cssm_nogate_desc* d, const cssm_nogate_weights* w, void* plan,
                          size_t plan_bytes, void* stream) {
  int s = nogate_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->kernel || !plan) return CSSM_ERR_NULL;
  if (!aligned16(plan)) return CSSM_ERR_ALIGN;
  if (plan_bytes < nogate_khat_bytes(*d)) return CSSM_ERR_WORKSPACE;
  // squashed like the gated block's K_hat but without the 1e-7 floor: the reference scans in
  // plain complex arithmetic here (direct_scalar_scan_op), not in log space
  return launch_khat(w->kernel, (cf*)plan, d->C, d->kernel_size, d->H, d->W, d->spectral_rho, 1, 0,
                     spectral_path(d->H, d->W), (cudaStream_t)stream);
}

int cssm_nogate_forward(const cssm_nogate_desc* d, const cssm_nogate_weights* w, const void* plan,
                        const float* x, float* y, void* workspace, size_t workspace_bytes,
                        void* stream) {
  int s = nogate_validate(d);
  if (s != CSSM_OK) return s;
  if (!w || !w->out_proj_kernel || !w->out_proj_bias || !plan || !x || !y || !workspace) return CSSM_ERR_NULL;
  if (!aligned16(plan) || !aligned16(x) || !aligned16(y) || !aligned16(workspace)) return CSSM_ERR_ALIGN;
  if (workspace_bytes < cssm_nogate_workspace_bytes(d)) return CSSM_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  float* planar = (float*)workspace;
  const int frames = d->B * d->T, HW = d->H * d->W;
  const long long tiles = (long long)frames * ((HW + 31) / 32) * ((d->C + 31) / 32);
  if (tiles > 0x7fffffffLL) return CSSM_ERR_DIMS;
  cl_to_planar_kernel<<<(unsigned)tiles, 256, 0, st>>>(x, planar, frames, HW, d->C);
  if ((s = check_launch()) != CSSM_OK) return s;
  s = launch_spectral(d->B, d->T, d->H, d->W, d->C, (const cf*)plan, nullptr, planar, 0, 1, st);
  if (s != CSSM_OK) return s;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = frames * HW; g.N = d->C; g.K = d->C; g.HW = HW;
  g.A = planar; g.a_planes = 2 * d->C; g.a_plane0 = 0;
  g.Wk = w->out_proj_kernel; g.bias = w->out_proj_bias;
  g.out = y; g.sub = x;
  g.T = d->T; g.H = d->H; g.W = d->W;
  return launch_gemm<true, false>(g, st);
}

}  // extern "C"
