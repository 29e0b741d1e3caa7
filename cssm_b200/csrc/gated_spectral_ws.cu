// Warp-specialised, pipelined version of the 64x64 fused gated spectral kernel.
//
// One CTA per (batch, channel) pair, 896 threads = 7 warpgroups:
//   warps  0- 7  A : forward row FFTs of step t (two real rows per complex FFT) -> ZR ring
//   warps  8-15  C : inverse row FFTs of step t, * staged SiLU(z) plane, store y
//   warps 16-24  B : forward column FFTs, gated recurrence (state in registers), inverse
//                    column FFTs -> GB ring; the only stage that is sequential in t
//   warp  25     L : TMA bulk copies of the x_main / SiLU(z) planes into 2-deep rings
//   warps 26-27    : idle (warpgroup padding for setmaxnreg)
// The three compute stages work on different steps at the same time (A runs ahead of B, C
// behind it); hand-over is by mbarriers (full / empty per ring slot), all waits bounded.
// Registers are re-balanced with setmaxnreg: A and C warps give registers up, B warps (state +
// gate maps) take them.
#include "r64.cuh"
#include "kernels.cuh"
#include "tc05.cuh"

namespace cssm {

constexpr int WS_THREADS = 896;
constexpr int WS_EX_CF = 25 * 4 * EX_GROUP_STRIDE;                 // exchange scratch, warps 0..24
constexpr int WS_SMEM_BYTES = (WS_EX_CF + 2 * R64_ZR_CF + 2 * R64_GB_CF) * 8 + 4 * 4096 * 4;

__device__ int g_ws_error = 0;      // first bounded wait that expired (role * 10 + site), 0 = none

// Register re-balancing.  setmaxnreg.inc blocks until the CTA's own pool (threads x registers at
// launch) has the registers, so the totals below must fit that pool or the kernel never ends:
// 16 A/C warps at WS_REG_AC + 12 B-group warps at WS_REG_B <= 28 warps at WS_REG_LAUNCH.
constexpr int WS_REG_LAUNCH = 72, WS_REG_AC = 56, WS_REG_B = 88;
static_assert(16 * WS_REG_AC + 12 * WS_REG_B <= 28 * WS_REG_LAUNCH, "setmaxnreg pool exceeded");

#ifndef CSSM_WS_SETMAXNREG
#define CSSM_WS_SETMAXNREG 1
#endif
template <int REGS> __device__ __forceinline__ void reg_dec() {
#if CSSM_WS_SETMAXNREG
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
#endif
}
template <int REGS> __device__ __forceinline__ void reg_inc() {
#if CSSM_WS_SETMAXNREG
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
#endif
}

// bounded wait whose outcome is the same for every lane of the warp (so a warp leaves its loop
// as a whole and never strands lanes at a __syncwarp)
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity) {
  const bool ok = tc::mbar_wait(bar, parity);
  return __all_sync(0xffffffffu, ok);
}

// one elected lane per warp arrives after the whole warp is done with the slot
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) tc::mbar_arrive(bar);
}

__global__ void __launch_bounds__(WS_THREADS, 1)
gated_spectral_r64_ws(float* __restrict__ xz, const cf* __restrict__ khat,
                      const float4* __restrict__ gates, int T, int C) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  cf* EX = reinterpret_cast<cf*>(smem_raw);
  cf* ZRr = EX + WS_EX_CF;                       // [2][R64_ZR_CF]
  cf* GBr = ZRr + 2 * R64_ZR_CF;                 // [2][R64_GB_CF]
  float* xbuf = reinterpret_cast<float*>(GBr + 2 * R64_GB_CF);   // [2][4096]
  float* zbuf = xbuf + 2 * 4096;                                 // [2][4096]
  // barriers: 0-1 xfull, 2-3 xempty, 4-5 zfull, 6-7 zempty, 8-9 zrfull, 10-11 zrempty,
  //           12-13 gbfull, 14-15 gbempty
  __shared__ __align__(8) uint64_t bars[16];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / C, ch = blockIdx.x % C;
  constexpr int HW = 4096;
  const size_t fstride = (size_t)2 * C * HW;
  float* x0 = xz + ((size_t)(b * T) * 2 * C + ch) * HW;          // x_main plane of step 0

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars[0 + i], 1);  tc::mbar_init(&bars[2 + i], 8);    // x: TMA / 8 A warps
      tc::mbar_init(&bars[4 + i], 1);  tc::mbar_init(&bars[6 + i], 8);    // z: TMA / 8 C warps
      tc::mbar_init(&bars[8 + i], 8);  tc::mbar_init(&bars[10 + i], 9);   // ZR: A warps / B warps
      tc::mbar_init(&bars[12 + i], 9); tc::mbar_init(&bars[14 + i], 8);   // GB: B warps / C warps
    }
    tc::fence_mbar_init();
  }
  __syncthreads();

  const int sub = lane & 3, a = lane >> 2;
  cf tw[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float s, co;
    sincospif(-(float)(a * k) / 32.0f, &s, &co);
    tw[k] = mk(co, s);
  }

  if (warp < 8) {
    // ============================== A: forward rows ==============================
    reg_dec<WS_REG_AC>();
    const int grp = warp * 4 + sub;
    cf* exg = EX + (warp * 4 + sub) * EX_GROUP_STRIDE;
    const int soff = (2 * grp) * 64 + a;
    for (int t = 0; t < T; ++t) {
      const int s = t & 1, ph = (t >> 1) & 1;
      if (!wait_warp(&bars[0 + s], ph)) { atomicExch(&g_ws_error, 11); break; }
      const float* xs = xbuf + s * 4096 + soff;
      cf v[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) v[m] = mk(xs[8 * m], xs[64 + 8 * m]);
      warp_arrive(&bars[2 + s], lane);                         // x slot free
      fft64_lane8<false>(v, tw, exg, a);
      if (!wait_warp(&bars[10 + s], ph ^ 1)) { atomicExch(&g_ws_error, 12); break; }
      cf* ZR = ZRr + s * R64_ZR_CF;
#pragma unroll
      for (int k2 = 0; k2 < 8; ++k2) ZR[grp * R64_ZRS + a + 8 * k2] = v[k2];
      warp_arrive(&bars[8 + s], lane);                         // ZR slot full
    }
  } else if (warp < 16) {
    // ============================== C: inverse rows ==============================
    reg_dec<WS_REG_AC>();
    const int wr = warp - 8;
    const int grp = wr * 4 + sub;
    cf* exg = EX + (warp * 4 + sub) * EX_GROUP_STRIDE;
    const int soff = (2 * grp) * 64 + a;
    for (int t = 0; t < T; ++t) {
      const int s = t & 1, ph = (t >> 1) & 1;
      if (!wait_warp(&bars[12 + s], ph)) { atomicExch(&g_ws_error, 21); break; }
      const cf* ge = GBr + s * R64_GB_CF + (2 * grp) * R64_GBS;
      const cf* go = ge + R64_GBS;
      cf v[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const int n = a + 8 * m;
        const int k = n <= 32 ? n : 64 - n;
        cf e = ge[k], o = go[k];
        if ((m == 0 || m == 4) && a == 0) { e.y = 0.f; o.y = 0.f; }
        v[m] = (n <= 32) ? mk(e.x - o.y, e.y + o.x) : mk(e.x + o.y, o.x - e.y);
      }
      warp_arrive(&bars[14 + s], lane);                        // GB slot free
      fft64_lane8<true>(v, tw, exg, a);
      if (!wait_warp(&bars[4 + s], ph)) { atomicExch(&g_ws_error, 22); break; }
      const float* zs = zbuf + s * 4096 + soff;
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1) v[n1] = mk(v[n1].x * zs[8 * n1], v[n1].y * zs[64 + 8 * n1]);
      warp_arrive(&bars[6 + s], lane);                         // z slot free
      float* y0 = x0 + (size_t)t * fstride + soff;
#pragma unroll
      for (int n1 = 0; n1 < 8; ++n1) {
        y0[8 * n1] = v[n1].x;
        y0[64 + 8 * n1] = v[n1].y;
      }
    }
  } else {
    reg_inc<WS_REG_B>();
    if (warp < 25) {
      // ====================== B: columns + gated recurrence ======================
      const int wr = warp - 16;
      const int grp = wr * 4 + sub;                  // half-spectrum column kw
      const bool col_on = grp <= 32;
      cf* exg = EX + (warp * 4 + sub) * EX_GROUP_STRIDE;
      const cf* khp = khat + (size_t)ch * (64 * 33) + (grp << 3) + a;
      const int par = a & 1, ph2 = a >> 1;
      const int kneg = (64 - grp) & 63;
      cf hst[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) hst[q] = mk(0.f, 0.f);
      for (int t = 0; t < T; ++t) {
        const int s = t & 1, ph = (t >> 1) & 1;
        const size_t frame = (size_t)(b * T + t);
        float4 g[8];
        cf kh[8];
        const float4* gp = gates + frame * (64 * 33) + (grp << 3) + a;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          g[q] = col_on ? __ldg(gp + q * (33 * 8)) : make_float4(0.f, 0.f, 0.f, 0.f);
          kh[q] = col_on ? khp[q * (33 * 8)] : mk(0.f, 0.f);
        }
        if (!wait_warp(&bars[8 + s], ph)) { atomicExch(&g_ws_error, 31); break; }
        const cf* ZR = ZRr + s * R64_ZR_CF;
        cf v[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const cf z1 = ZR[(ph2 + 4 * m) * R64_ZRS + grp];
          const cf z2 = ZR[(ph2 + 4 * m) * R64_ZRS + kneg];
          v[m] = par ? mk(0.5f * (z1.y + z2.y), 0.5f * (z2.x - z1.x))
                     : mk(0.5f * (z1.x + z2.x), 0.5f * (z1.y - z2.y));
        }
        warp_arrive(&bars[10 + s], lane);                      // ZR slot free
        fft64_lane8<false>(v, tw, exg, a);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const cf A = mk(kh[q].x * g[q].x, kh[q].y * g[q].x);
          cf U = mk(g[q].y * v[q].x, g[q].y * v[q].y);
          if (U.x * U.x + U.y * U.y < g[q].w * g[q].w) U = mk(g[q].w, 0.f);
          cf h = cmul(A, hst[q]);
          h.x += U.x; h.y += U.y;
          hst[q] = h;
          v[q] = mk(g[q].z * h.x, g[q].z * h.y);
        }
        fft64_lane8<true>(v, tw, exg, a);
        if (!wait_warp(&bars[14 + s], ph ^ 1)) { atomicExch(&g_ws_error, 32); break; }
        cf* GB = GBr + s * R64_GB_CF;
#pragma unroll
        for (int n1 = 0; n1 < 8; ++n1)
          if (col_on) GB[(a + 8 * n1) * R64_GBS + grp] = v[n1];
        warp_arrive(&bars[12 + s], lane);                      // GB slot full
      }
    } else if (warp == 25) {
      // ============================== L: TMA loader ==============================
      if (lane == 0) {
        for (int t = 0; t < T; ++t) {
          const int s = t & 1, ph = (t >> 1) & 1;
          const float* xs = x0 + (size_t)t * fstride;
          if (!tc::mbar_wait(&bars[2 + s], ph ^ 1)) { atomicExch(&g_ws_error, 41); break; }
          tc::fence_proxy_async();
          tc::mbar_expect_tx(&bars[0 + s], 16384);
          tc::bulk_g2s(xbuf + s * 4096, xs, 16384, &bars[0 + s]);
          if (!tc::mbar_wait(&bars[6 + s], ph ^ 1)) { atomicExch(&g_ws_error, 42); break; }
          tc::fence_proxy_async();
          tc::mbar_expect_tx(&bars[4 + s], 16384);
          tc::bulk_g2s(zbuf + s * 4096, xs + (size_t)C * HW, 16384, &bars[4 + s]);
        }
      }
      __syncwarp();
    }
  }
}

int read_ws_error(int* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_ws_error, sizeof(int));
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

int launch_gated_spectral_ws(float* xz, const cf* khat, const float* gates, int B, int T, int C,
                             cudaStream_t st) {
  // refuse to launch if the compiled register count makes the setmaxnreg pool too small
  cudaFuncAttributes fa;
  cudaError_t e = cudaFuncGetAttributes(&fa, gated_spectral_r64_ws);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  if (CSSM_WS_SETMAXNREG && 16 * WS_REG_AC + 12 * WS_REG_B > 28 * fa.numRegs) return CSSM_ERR_UNSUPPORTED;
  e = cudaFuncSetAttribute(gated_spectral_r64_ws,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, WS_SMEM_BYTES);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  gated_spectral_r64_ws<<<B * C, WS_THREADS, WS_SMEM_BYTES, st>>>(
      xz, khat, reinterpret_cast<const float4*>(gates), T, C);
  return check_launch();
}

}  // namespace cssm
