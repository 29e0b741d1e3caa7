// Pointwise / stencil / reduction kernels of the bf16 CSSM-SHViT forward (channels-last bf16
// activations, fp32 arithmetic), and the weight-packing kernels of its plan.
#include "kernels.cuh"
#include "bf16_ops.cuh"

namespace cssm {

// ------------------------------------------------------------------ plan: weight packing ----
// src (K, N) fp32 row-major (a Dense kernel, or an HWIO conv kernel flattened over its taps and
// input channels) -> dst (N, ldw) bf16, K-major, zero padded to ldw, column n scaled by
// colscale[n] (BatchNorm fold, temporal tap of the mixer) when given.
__global__ void pack_wt_kernel(const float* __restrict__ src, int K, int N, const float* __restrict__ colscale,
                               __nv_bfloat16* __restrict__ dst, int ldw) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * ldw) return;
  const int n = i / ldw, k = i - n * ldw;
  float v = 0.f;
  if (k < K) {
    v = src[(size_t)k * N + n];
    if (colscale) v *= colscale[n];
  }
  dst[i] = __float2bfloat16(v);
}
int launch_pack_wt(const float* src, int K, int N, const float* colscale, __nv_bfloat16* dst, int ldw,
                   cudaStream_t st) {
  const int n = N * ldw;
  pack_wt_kernel<<<(n + 255) / 256, 256, 0, st>>>(src, K, N, colscale, dst, ldw);
  return check_launch();
}

// 3x3 conv kernel with 32 input channels in the wide-pixel layout: src HWIO (3,3,32,N) fp32 ->
// dst (N, 384) bf16 with k = row*128 + p*64 + j: j < 32 is column 2p, channel j; j >= 32 is column
// 2p+1, channel j-32 (zero for the non-existent column 3).
__global__ void pack_conv_wide_kernel(const float* __restrict__ src, int N, const float* __restrict__ colscale,
                                      __nv_bfloat16* __restrict__ dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * 384) return;
  const int n = i / 384, k = i - n * 384;
  const int ti = k >> 7, p = (k >> 6) & 1, j = k & 63;
  const int tj = 2 * p + (j >> 5), c = j & 31;
  float v = 0.f;
  if (tj < 3) {
    v = src[(size_t)((ti * 3 + tj) * 32 + c) * N + n];
    if (colscale) v *= colscale[n];
  }
  dst[i] = __float2bfloat16(v);
}
// Packs an HWIO 3x3 kernel for the stride-2 conv of an input of width Wi (see conv3x3s2_weight_layout).
int launch_pack_conv3x3(const float* src, int Cin, int N, int Wi, const float* colscale, __nv_bfloat16* dst,
                        cudaStream_t st) {
  if (conv3x3s2_weight_layout(Cin, Wi, N)) {
    pack_conv_wide_kernel<<<(N * 384 + 255) / 256, 256, 0, st>>>(src, N, colscale, dst);
    return check_launch();
  }
  const int K = 9 * Cin;
  return launch_pack_wt(src, K, N, colscale, dst, (K + 63) / 64 * 64, st);
}

// BatchNorm (running statistics, eps 1e-5) after a bias-free conv as a per-channel scale and bias
__global__ void bn_fold_kernel(const float* scale, const float* bias, const float* mean, const float* var,
                               int C, float* oscale, float* obias) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float s = scale[c] * rsqrtf(var[c] + 1e-5f);
  oscale[c] = s;
  obias[c] = bias[c] - mean[c] * s;
}
int launch_bn_fold(const float* scale, const float* bias, const float* mean, const float* var, int C,
                   float* oscale, float* obias, cudaStream_t st) {
  bn_fold_kernel<<<(C + 127) / 128, 128, 0, st>>>(scale, bias, mean, var, C, oscale, obias);
  return check_launch();
}

// out[c] = a[c] * s[c] + b[c]   (bias of the in_proj with the T = 1 temporal tap folded in)
__global__ void affine_vec_kernel(const float* a, const float* s, const float* b, int C, float* out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) out[c] = (s ? a[c] * s[c] : a[c]) + (b ? b[c] : 0.f);
}
int launch_affine_vec(const float* a, const float* s, const float* b, int C, float* out, cudaStream_t st) {
  affine_vec_kernel<<<(C + 127) / 128, 128, 0, st>>>(a, s, b, C, out);
  return check_launch();
}

__global__ void fill_kernel(float* p, int n, float v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}
int launch_fill(float* p, int n, float v, cudaStream_t st) {
  fill_kernel<<<(n + 127) / 128, 128, 0, st>>>(p, n, v);
  return check_launch();
}

// out[k, n] = src[k, n] * s[n], float32 (the first stem conv keeps float32 weights)
__global__ void scale_cols_kernel(const float* __restrict__ src, int K, int N, const float* __restrict__ s,
                                  float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < K * N) out[i] = src[i] * s[i % N];
}
int launch_scale_cols(const float* src, int K, int N, const float* s, float* out, cudaStream_t st) {
  scale_cols_kernel<<<(K * N + 255) / 256, 256, 0, st>>>(src, K, N, s, out);
  return check_launch();
}

// ------------------------------------------------------------------ first stem conv ----
// 3x3 stride-2 'SAME' conv of the image (few input channels), BatchNorm folded, GELU.
// x (Nimg, Hi, Wi, Cin) bf16 -> y (Nimg, Ho, Wo, Co) bf16.  wk (9*Cin, Co) fp32 already scaled by the
// BatchNorm factor, bias (Co).  Thread = one output pixel and CO output channels: the weights are
// read from shared memory as float4 broadcasts (every thread of a warp reads the same address).
template <int CO>
__global__ void __launch_bounds__(128)
stem_conv1_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wk,
                  const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int Nimg, int Hi,
                  int Wi, int Cin, int Ho, int Wo, int Co, int pad_h, int pad_w, int gelu) {
  extern __shared__ __align__(16) float ws[];      // (9*Cin, Co) + (Co)
  const int K = 9 * Cin;
  for (int i = threadIdx.x; i < K * Co; i += blockDim.x) ws[i] = wk[i];
  for (int i = threadIdx.x; i < Co; i += blockDim.x) ws[K * Co + i] = bias[i];
  __syncthreads();
  const int groups = Co / CO;
  const long long total = (long long)Nimg * Ho * Wo * groups;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total;
       it += (long long)gridDim.x * blockDim.x) {
    // consecutive threads = consecutive pixels (the channel group is the slow index)
    const long long px = it % ((long long)Nimg * Ho * Wo);
    const int cg = (int)(it / ((long long)Nimg * Ho * Wo));
    const int wo = (int)(px % Wo), ho = (int)((px / Wo) % Ho), n = (int)(px / ((long long)Wo * Ho));
    float acc[CO];
#pragma unroll
    for (int j = 0; j < CO; ++j) acc[j] = ws[K * Co + cg * CO + j];
    for (int ti = 0; ti < 3; ++ti) {
      const int hi = ho * 2 + ti - pad_h;
      if (hi < 0 || hi >= Hi) continue;
      for (int tj = 0; tj < 3; ++tj) {
        const int wi = wo * 2 + tj - pad_w;
        if (wi < 0 || wi >= Wi) continue;
        const __nv_bfloat16* xp = x + (((size_t)n * Hi + hi) * Wi + wi) * Cin;
        for (int c = 0; c < Cin; ++c) {
          const float xv = __bfloat162float(xp[c]);
          const float4* wr = reinterpret_cast<const float4*>(ws + ((ti * 3 + tj) * Cin + c) * Co + cg * CO);
#pragma unroll
          for (int j = 0; j < CO / 4; ++j) {
            const float4 w4 = wr[j];
            acc[4 * j] = fmaf(xv, w4.x, acc[4 * j]); acc[4 * j + 1] = fmaf(xv, w4.y, acc[4 * j + 1]);
            acc[4 * j + 2] = fmaf(xv, w4.z, acc[4 * j + 2]); acc[4 * j + 3] = fmaf(xv, w4.w, acc[4 * j + 3]);
          }
        }
      }
    }
    if (gelu) {
#pragma unroll
      for (int j = 0; j < CO; ++j) acc[j] = gelu_tanh_f(acc[j]);
    }
    uint4* yo = reinterpret_cast<uint4*>(y + (size_t)px * Co + cg * CO);
#pragma unroll
    for (int j = 0; j < CO / 8; ++j) {
      const float v8[8] = {acc[8 * j], acc[8 * j + 1], acc[8 * j + 2], acc[8 * j + 3],
                           acc[8 * j + 4], acc[8 * j + 5], acc[8 * j + 6], acc[8 * j + 7]};
      yo[j] = pack8(v8);
    }
  }
}
// The same conv for the shape the model has (3 input channels, 32 output channels, even image sides:
// XLA's 'SAME' rule then pads one row below and one column to the right only).  Thread = TWO adjacent
// output pixels: their 3 x 5 x 3 input window is loaded once with 8-byte loads, every weight vector
// read from shared memory (float4 broadcasts) feeds both pixels, the 32 output channels of a pixel are
// 16 packed f32x2 accumulators (half the FMA issue slots of scalar code), GELU on pairs, and the
// thread writes 128 contiguous bytes.
__global__ void __launch_bounds__(128)
stem_conv1_pair_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wk,
                       const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int Nimg, int Hi,
                       int Wi, int Ho, int Wo, int gelu) {
  constexpr int CI = 3, CO = 32, K = 9 * CI;
  __shared__ __align__(16) float ws[K * CO + CO];
  for (int i = threadIdx.x; i < K * CO; i += blockDim.x) ws[i] = wk[i];
  for (int i = threadIdx.x; i < CO; i += blockDim.x) ws[K * CO + i] = bias[i];
  __syncthreads();
  const int Wp = Wo / 2;
  const long long total = (long long)Nimg * Ho * Wp;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total;
       it += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(it % Wp), ho = (int)((it / Wp) % Ho), n = (int)(it / ((long long)Wp * Ho));
    // window: rows 2 ho .. 2 ho + 2, columns 4 p .. 4 p + 4 (row Hi / column Wi = zero padding)
    float in[3][5 * CI];
#pragma unroll
    for (int ti = 0; ti < 3; ++ti) {
      const int hi = 2 * ho + ti;
      const bool rin = hi < Hi;
      const uint2* rp = reinterpret_cast<const uint2*>(x + (((size_t)n * Hi + (rin ? hi : 0)) * Wi + 4 * p) * CI);
      const bool c4 = 4 * p + 4 < Wi;
      uint2 u[4];
#pragma unroll
      for (int q = 0; q < 3; ++q) u[q] = rin ? __ldg(rp + q) : make_uint2(0u, 0u);
      u[3] = (rin && c4) ? __ldg(rp + 3) : make_uint2(0u, 0u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = bf16x2_to_float2(u[q].x), b = bf16x2_to_float2(u[q].y);
        if (4 * q < 5 * CI) in[ti][4 * q] = a.x;
        if (4 * q + 1 < 5 * CI) in[ti][4 * q + 1] = a.y;
        if (4 * q + 2 < 5 * CI) in[ti][4 * q + 2] = b.x;
        if (4 * q + 3 < 5 * CI) in[ti][4 * q + 3] = b.y;
      }
    }
    unsigned long long accA[CO / 2], accB[CO / 2];
#pragma unroll
    for (int j = 0; j < CO / 2; ++j) {
      const float2 b2 = *reinterpret_cast<const float2*>(ws + K * CO + 2 * j);
      accA[j] = accB[j] = pk2(b2.x, b2.y);
    }
#pragma unroll
    for (int ti = 0; ti < 3; ++ti)
#pragma unroll
      for (int tj = 0; tj < 3; ++tj)
#pragma unroll
        for (int c = 0; c < CI; ++c) {
          const float xa = in[ti][tj * CI + c], xb = in[ti][(tj + 2) * CI + c];
          const unsigned long long pa = pk2(xa, xa), pb = pk2(xb, xb);
          const float4* wr = reinterpret_cast<const float4*>(ws + ((ti * 3 + tj) * CI + c) * CO);
#pragma unroll
          for (int j = 0; j < CO / 4; ++j) {
            const float4 w4 = wr[j];
            const unsigned long long w01 = pk2(w4.x, w4.y), w23 = pk2(w4.z, w4.w);
            accA[2 * j] = fma2(pa, w01, accA[2 * j]); accA[2 * j + 1] = fma2(pa, w23, accA[2 * j + 1]);
            accB[2 * j] = fma2(pb, w01, accB[2 * j]); accB[2 * j + 1] = fma2(pb, w23, accB[2 * j + 1]);
          }
        }
    uint4* yo = reinterpret_cast<uint4*>(y + ((((size_t)n * Ho + ho) * Wo) + 2 * p) * CO);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int j = 0; j < CO / 8; ++j) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float a, b;
          upk2(half ? accB[4 * j + e] : accA[4 * j + e], a, b);
          if (gelu) gelu_tanh_x2(a, b);
          o[e] = float2_to_bf16x2(a, b);
        }
        yo[half * (CO / 8) + j] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// The same conv once more for that shape, on the tensor cores: warp-level mma.sync (m16n8k16, bf16 in,
// f32 accumulate) -- the contraction is K = 27, far too short for a tcgen05 pipeline (a 128 x 32 tile
// per barrier round trip was measured at 390 us against the 328 us of the packed-FMA kernel above).
// A warp owns 16 consecutive output pixels of one row x all 32 channels.  K is laid out as three
// window rows of ten slots (nine taps*channels + one zero-weight pad), so that every A-fragment
// register is one ALIGNED 32-bit word of the image: window row ti of pixel wo starts at element
// 6 wo of image row 2 ho + ti, and lane (g, t) needs words t, t + 4, t + 8, t + 12 of the 15-word
// patch of pixels g and g + 8 -- eight coalesced loads per lane and tile, no shuffles.  The weights
// (B fragments) and the bias live in registers.  Epilogue: bias, GELU, bf16; the quad's words pass
// through a per-warp shared-memory patch so that every lane stores 16 contiguous bytes.
constexpr int SM_WARPS = 8;
__global__ void __launch_bounds__(SM_WARPS * 32, 3)
stem_conv1_mma_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wk,
                      const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int Nimg, int Hi, int Wi,
                      int Ho, int Wo, int gelu) {
  __shared__ __align__(16) uint32_t stage[SM_WARPS][16 * 20];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  // B fragments: slot k = 16 s + 2 t + 8 h (+0, +1) of output channel n = 8 nt + g
  uint32_t bf[4][2][2];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int sk = 0; sk < 2; ++sk)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float wv[2];
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int k = 16 * sk + 2 * t + 8 * h + e2, ti = k / 10, e = k - ti * 10;
          wv[e2] = (ti < 3 && e < 9) ? __ldg(wk + (ti * 9 + e) * 32 + nt * 8 + g) : 0.f;
        }
        bf[nt][sk][h] = float2_to_bf16x2(wv[0], wv[1]);
      }
  float2 bz[4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) bz[nt] = __ldg(reinterpret_cast<const float2*>(bias + nt * 8 + 2 * t));
  // the lane's four words of a patch: word w = t + 4 i -> window row w / 5, word w % 5 of it (15 = none)
  int wti[4], wj[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { const int w = t + 4 * i; wti[i] = w / 5; wj[i] = w - wti[i] * 5; }
  const uint32_t* xw = reinterpret_cast<const uint32_t*>(x);
  const int tpr = Wo / 16;                               // tiles per output row
  const long long ntiles = (long long)Nimg * Ho * tpr;
  // a warp walks a contiguous range of tiles (row after row of one image: the image row shared by two
  // output rows is still in L1), its coordinates advanced without divisions
  const long long nwarps = (long long)gridDim.x * SM_WARPS, gw = (long long)blockIdx.x * SM_WARPS + warp;
  const long long per = (ntiles + nwarps - 1) / nwarps;
  long long tile = gw * per;
  const long long tend = tile + per < ntiles ? tile + per : ntiles;
  // word offsets of the lane's eight patch words from the first word of the tile's window
  int woff[2][4];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh)
#pragma unroll
    for (int i = 0; i < 4; ++i) woff[hh][i] = ((wti[i] * Wi + 2 * (g + 8 * hh)) * 3 >> 1) + wj[i];
  auto fetch = [&](bool live, long long base, int ho, int wt, uint32_t (&a)[2][4]) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const bool v2 = 2 * (wt * 16 + g + 8 * hh) + 2 < Wi;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool ok = live && wti[i] < 3 && 2 * ho + wti[i] < Hi && (wj[i] < 3 || v2);
        uint32_t u = 0u;
        if (ok) u = __ldg(xw + base + woff[hh][i]);
        if (wj[i] == 4) u &= 0xFFFFu;                     // the upper half belongs to the next pixel
        a[hh][i] = u;
      }
    }
  };
  // coordinates of `tile`: (image * Ho + ho) = rowi, tile of the row wt; window word base
  long long rowi = tile < ntiles ? tile / tpr : 0;
  int wt = (int)(tile < ntiles ? tile - rowi * tpr : 0);
  int ho = (int)(rowi % Ho);
  long long b_ = rowi / Ho;
  auto base_of = [&](long long bb, int h, int w) { return ((bb * Hi + 2 * h) * Wi + 32 * w) * 3 >> 1; };
  uint32_t cur[2][4], nxt[2][4];
  fetch(tile < tend, base_of(b_, ho, wt), ho, wt, cur);
  for (; tile < tend; ++tile) {
    // coordinates of the next tile
    int wt2 = wt + 1, ho2 = ho;
    long long b2 = b_, rowi2 = rowi;
    if (wt2 == tpr) { wt2 = 0; ++rowi2; if (++ho2 == Ho) { ho2 = 0; ++b2; } }
    fetch(tile + 1 < tend, base_of(b2, ho2, wt2), ho2, wt2, nxt);
    float c[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { c[nt][0] = bz[nt].x; c[nt][1] = bz[nt].y; c[nt][2] = bz[nt].x; c[nt][3] = bz[nt].y; }
    // A fragment of k-step s: {row g: word t + 8 s, row g + 8: same, row g: word t + 8 s + 4, row g + 8: same}
#pragma unroll
    for (int sk = 0; sk < 2; ++sk)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[nt][0]), "+f"(c[nt][1]), "+f"(c[nt][2]), "+f"(c[nt][3])
            : "r"(cur[0][2 * sk]), "r"(cur[1][2 * sk]), "r"(cur[0][2 * sk + 1]), "r"(cur[1][2 * sk + 1]),
              "r"(bf[nt][sk][0]), "r"(bf[nt][sk][1]));
    uint32_t* sp = stage[warp];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      if (gelu) { gelu_tanh_x2(c[nt][0], c[nt][1]); gelu_tanh_x2(c[nt][2], c[nt][3]); }
      sp[g * 20 + 4 * nt + t] = float2_to_bf16x2(c[nt][0], c[nt][1]);
      sp[(g + 8) * 20 + 4 * nt + t] = float2_to_bf16x2(c[nt][2], c[nt][3]);
    }
    __syncwarp();
    __nv_bfloat16* yo = y + ((rowi * Wo + wt * 16) * 32);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int p = (lane >> 2) + 8 * hh;
      *reinterpret_cast<uint4*>(yo + p * 32 + (lane & 3) * 8) = *reinterpret_cast<const uint4*>(sp + p * 20 + (lane & 3) * 4);
    }
    __syncwarp();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
      for (int i = 0; i < 4; ++i) cur[hh][i] = nxt[hh][i];
    wt = wt2; ho = ho2; b_ = b2; rowi = rowi2;
  }
}

int launch_stem_conv1(const __nv_bfloat16* x, const float* wk, const float* bias, __nv_bfloat16* y,
                      int Nimg, int Hi, int Wi, int Cin, int Co, int gelu, cudaStream_t st) {
  if (Co % 8 != 0 || Cin > 16) return CSSM_ERR_UNSUPPORTED;
  const int Ho = (Hi + 1) / 2, Wo = (Wi + 1) / 2;
  const int pad_h = ((Ho - 1) * 2 + 3 - Hi > 0 ? (Ho - 1) * 2 + 3 - Hi : 0) / 2;
  const int pad_w = ((Wo - 1) * 2 + 3 - Wi > 0 ? (Wo - 1) * 2 + 3 - Wi : 0) / 2;
  if (Cin == 3 && Co == 32 && Hi % 2 == 0 && Wi % 32 == 0 && aligned16(x) && aligned16(y) && aligned16(bias)) {
    const long long tiles = (long long)Nimg * Ho * (Wo / 16);
    long long blocks = (tiles + SM_WARPS - 1) / SM_WARPS;
    if (blocks > 148 * 3) blocks = 148 * 3;                // one wave at three resident blocks per SM
    stem_conv1_mma_kernel<<<(int)blocks, SM_WARPS * 32, 0, st>>>(x, wk, bias, y, Nimg, Hi, Wi, Ho, Wo, gelu);
    return check_launch();
  }
  if (Cin == 3 && Co == 32 && Hi % 2 == 0 && Wi % 4 == 0 && aligned16(x) && aligned16(y)) {
    const long long pairs = (long long)Nimg * Ho * (Wo / 2);
    long long blocks = (pairs + 127) / 128;
    if (blocks > 148 * 16) blocks = 148 * 16;
    stem_conv1_pair_kernel<<<(int)blocks, 128, 0, st>>>(x, wk, bias, y, Nimg, Hi, Wi, Ho, Wo, gelu);
    return check_launch();
  }
  const size_t smem = (size_t)(9 * Cin * Co + Co) * 4;
  const int co = Co % 32 == 0 ? 32 : (Co % 16 == 0 ? 16 : 8);
  const long long total = (long long)Nimg * Ho * Wo * (Co / co);
  long long blocks = (total + 127) / 128;
  if (blocks > 148 * 32) blocks = 148 * 32;
  auto kern = co == 32 ? stem_conv1_kernel<32> : (co == 16 ? stem_conv1_kernel<16> : stem_conv1_kernel<8>);
  kern<<<(int)blocks, 128, smem, st>>>(x, wk, bias, y, Nimg, Hi, Wi, Cin, Ho, Wo, Co, pad_h, pad_w, gelu);
  return check_launch();
}

// ------------------------------------------------------------------ depthwise conv ----
// Depthwise KS x KS 'SAME' conv (zero padding) on channels-last bf16, thread = (strip of RH output
// rows of one column, 8 channels): every input value of the strip's (RH + KS - 1) x KS window is
// loaded once and feeds up to RH outputs.
//   v    = pre ? pre_a[n, c] * x + pre_b[n, c] : x          (LayerNorm over a whole sample, applied on load)
//   out  = (add_centre ? v_centre : 0) + sum_taps w * v + bias;  then GELU when gelu != 0.
template <int KS, int RH>
__global__ void __launch_bounds__(256)
dwconv_cl_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wk,
                 const float* __restrict__ bias, const float* __restrict__ pre_a,
                 const float* __restrict__ pre_b, __nv_bfloat16* __restrict__ y, float* __restrict__ y_f32,
                 int Nimg, int H, int W, int C, int add_centre, int gelu) {
  extern __shared__ float ws[];                    // (KS*KS, C) + (C)
  for (int i = threadIdx.x; i < KS * KS * C; i += blockDim.x) ws[i] = wk ? wk[i] : 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) ws[KS * KS * C + i] = (wk && bias) ? bias[i] : 0.f;
  __syncthreads();
  constexpr int P = (KS - 1) / 2;
  const int groups = C / 8, strips = (H + RH - 1) / RH;
  const long long total = (long long)Nimg * strips * W * groups;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total;
       it += (long long)gridDim.x * blockDim.x) {
    const int cg = (int)(it % groups);
    long long r = it / groups;
    const int w = (int)(r % W); r /= W;
    const int sp = (int)(r % strips), n = (int)(r / strips);
    const int h0 = sp * RH, c0 = cg * 8;
    float pa[8], pb[8];
    if (pre_a != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { pa[j] = pre_a[(size_t)n * C + c0 + j]; pb[j] = pre_b[(size_t)n * C + c0 + j]; }
    }
    float acc[RH][8];
#pragma unroll
    for (int o = 0; o < RH; ++o)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[o][j] = ws[KS * KS * C + c0 + j];
    const __nv_bfloat16* xn = x + (size_t)n * H * W * C + c0;
#pragma unroll
    for (int ir = 0; ir < RH + KS - 1; ++ir) {
      const int hi = h0 + ir - P;
      if (hi < 0 || hi >= H) continue;
#pragma unroll
      for (int tj = 0; tj < KS; ++tj) {
        const int wi = w + tj - P;
        if (wi < 0 || wi >= W) continue;
        float v[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(xn + ((size_t)hi * W + wi) * C)), v);
        if (pre_a != nullptr) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = fmaf(pa[j], v[j], pb[j]);
        }
#pragma unroll
        for (int o = 0; o < RH; ++o) {
          const int ti = ir - o;                   // tap row that maps input row ir to output row o
          if (ti < 0 || ti >= KS) continue;
          const float* wr = ws + (ti * KS + tj) * C + c0;
          const float4 w0 = *reinterpret_cast<const float4*>(wr), w1 = *reinterpret_cast<const float4*>(wr + 4);
          acc[o][0] = fmaf(v[0], w0.x, acc[o][0]); acc[o][1] = fmaf(v[1], w0.y, acc[o][1]);
          acc[o][2] = fmaf(v[2], w0.z, acc[o][2]); acc[o][3] = fmaf(v[3], w0.w, acc[o][3]);
          acc[o][4] = fmaf(v[4], w1.x, acc[o][4]); acc[o][5] = fmaf(v[5], w1.y, acc[o][5]);
          acc[o][6] = fmaf(v[6], w1.z, acc[o][6]); acc[o][7] = fmaf(v[7], w1.w, acc[o][7]);
          if (add_centre && ti == P && tj == P) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[o][j] += v[j];
          }
        }
      }
    }
#pragma unroll
    for (int o = 0; o < RH; ++o) {
      const int h = h0 + o;
      if (h >= H) continue;
      if (gelu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[o][j] = gelu_tanh_f(acc[o][j]);
      }
      const size_t off = (((size_t)n * H + h) * W + w) * C + c0;
      if (y_f32 != nullptr) {
        *reinterpret_cast<float4*>(y_f32 + off) = make_float4(acc[o][0], acc[o][1], acc[o][2], acc[o][3]);
        *reinterpret_cast<float4*>(y_f32 + off + 4) = make_float4(acc[o][4], acc[o][5], acc[o][6], acc[o][7]);
      } else {
        *reinterpret_cast<uint4*>(y + off) = pack8(acc[o]);
      }
    }
  }
}

// Depthwise KS x KS 'SAME' conv, tiled through shared memory (the path of every bf16 output).
// A CTA of 128 threads owns a tile of 8 output rows x 16 columns x 64 channels of one image and one
// channel slice; the bf16 input patch with its halo is staged with 16-byte loads as it lies in
// memory ([row][column][channel]; the per-sample LayerNorm affine, when given, is applied while
// staging and the result rounded to bf16, zeros stay zeros outside the image).  Thread = one PAIR of
// channels of one column group (a warp = the 32 channel pairs of the slice), its KS*KS weight pairs in
// registers; for each of its four columns it walks the input rows of the window once: KS four-byte
// shared-memory loads per row (conflict-free: the lanes of a warp are consecutive pairs), each value
// pair feeds the output rows it belongs to with packed f32x2 FMAs (two channels per instruction).
// Tile geometry as template parameters: CG column groups (32 * CG threads), NC columns per group, TH rows;
// the launcher picks one that divides the plane (8 x 16 tiles on a 28 x 28 plane compute 31 % more
// outputs than the plane has).
template <int KS, int CG, int NC, int TH>
__global__ void __launch_bounds__(32 * CG)
dwconv_tiled_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wk,
                    const float* __restrict__ bias, const float* __restrict__ pre_a,
                    const float* __restrict__ pre_b, __nv_bfloat16* __restrict__ y, int H, int W, int C,
                    int add_centre, int gelu) {
  constexpr int CS = 64, P = (KS - 1) / 2, TW = CG * NC, PW = TW + KS - 1, PH = TH + KS - 1, NT = 32 * CG;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [PH][PW][CS]
  const int tiles_w = (W + TW - 1) / TW, tiles_h = (H + TH - 1) / TH, slices = C / CS;
  int bid = blockIdx.x;
  const int sl = bid % slices; bid /= slices;
  const int tr = bid % (tiles_w * tiles_h), n = bid / (tiles_w * tiles_h);
  const int h0 = (tr / tiles_w) * TH, w0 = (tr % tiles_w) * TW, cs0 = sl * CS;
  const int cp = threadIdx.x & 31, cgp = threadIdx.x >> 5;                 // channel pair, column group
  // stage the patch (zeros outside the image): asynchronous 16-byte copies, all in flight at once
  // (with the LayerNorm affine the values pass through registers instead)
  constexpr int CH = CS / 8;                         // 16-byte chunks per pixel of the slice
  const __nv_bfloat16* xn = x + (size_t)n * H * W * C + cs0;
  // the thread's chunk of eight channels is the same for every element it stages (NT is a multiple of
  // CH): its LayerNorm affine is fetched once, with four 16-byte loads
  float pav[8], pbv[8];
  if (pre_a != nullptr) {
    const int ck0 = threadIdx.x & (CH - 1);
    const float4* pa4 = reinterpret_cast<const float4*>(pre_a + (size_t)n * C + cs0 + ck0 * 8);
    const float4* pb4 = reinterpret_cast<const float4*>(pre_b + (size_t)n * C + cs0 + ck0 * 8);
    const float4 a0 = __ldg(pa4), a1 = __ldg(pa4 + 1), b0 = __ldg(pb4), b1 = __ldg(pb4 + 1);
    pav[0] = a0.x; pav[1] = a0.y; pav[2] = a0.z; pav[3] = a0.w; pav[4] = a1.x; pav[5] = a1.y; pav[6] = a1.z; pav[7] = a1.w;
    pbv[0] = b0.x; pbv[1] = b0.y; pbv[2] = b0.z; pbv[3] = b0.w; pbv[4] = b1.x; pbv[5] = b1.y; pbv[6] = b1.z; pbv[7] = b1.w;
  }
  if (pre_a == nullptr) {
    for (int pr = 0; pr < PH; ++pr) {
      const int hi = h0 + pr - P;
      const bool hin = hi >= 0 && hi < H;
      for (int q = threadIdx.x; q < PW * CH; q += NT) {
        const int ck = q & (CH - 1), pc = q / CH;
        const int wi = w0 + pc - P;
        const bool in = hin && wi >= 0 && wi < W;
        __nv_bfloat16* dst = tile + ((size_t)pr * PW + pc) * CS + ck * 8;
        const __nv_bfloat16* src = xn + ((size_t)(in ? hi : 0) * W + (in ? wi : 0)) * C + ck * 8;
        // src-size 0 writes zeros
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(in ? 16 : 0) : "memory");
      }
    }
  } else {
    // through registers, six 16-byte loads in flight per thread
    constexpr int TOT = PH * PW * CH, SBN = 6;
    for (int base = threadIdx.x; base < TOT; base += NT * SBN) {
      uint4 raw[SBN];
      bool inb[SBN];
#pragma unroll
      for (int u = 0; u < SBN; ++u) {
        const int i = base + u * NT;
        const int pr = i / (PW * CH), q = i - pr * (PW * CH);
        const int ck = q & (CH - 1), pc = q / CH;
        const int hi = h0 + pr - P, wi = w0 + pc - P;
        inb[u] = i < TOT && hi >= 0 && hi < H && wi >= 0 && wi < W;
        raw[u] = inb[u] ? __ldg(reinterpret_cast<const uint4*>(xn + ((size_t)hi * W + wi) * C + ck * 8))
                        : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < SBN; ++u) {
        const int i = base + u * NT;
        if (i >= TOT) continue;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (inb[u]) {
          float f[8];
          unpack8(raw[u], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = fmaf(pav[j], f[j], pbv[j]);
          v = pack8(f);
        }
        *reinterpret_cast<uint4*>(tile + (size_t)i * 8) = v;        // [pr][pc][ck] is the order of i
      }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  unsigned long long wr[KS * KS];
#pragma unroll
  for (int t = 0; t < KS * KS; ++t) {
    const float2 w2 = wk ? __ldg(reinterpret_cast<const float2*>(wk + (size_t)t * C + cs0) + cp) : make_float2(0.f, 0.f);
    wr[t] = pk2(w2.x + ((add_centre && t == P * KS + P) ? 1.0f : 0.f),
                w2.y + ((add_centre && t == P * KS + P) ? 1.0f : 0.f));     // x + conv(x)
  }
  const float2 b2 = (wk && bias) ? __ldg(reinterpret_cast<const float2*>(bias + cs0) + cp) : make_float2(0.f, 0.f);
  const unsigned long long bz = pk2(b2.x, b2.y);
  const uint32_t* tile32 = reinterpret_cast<const uint32_t*>(tile);        // [PH][PW][32 pairs]
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
#pragma unroll 1
  for (int cc = 0; cc < NC; ++cc) {
    const int wl = cgp * NC + cc;                    // column inside the tile
    if (w0 + wl >= W) break;
    unsigned long long acc[TH];
#pragma unroll
    for (int o = 0; o < TH; ++o) acc[o] = bz;
#pragma unroll
    for (int ir = 0; ir < PH; ++ir) {
      unsigned long long xv[KS];
#pragma unroll
      for (int tj = 0; tj < KS; ++tj) {
        const uint32_t u = tile32[((size_t)ir * PW + wl + tj) * 32 + cp];
        xv[tj] = pk2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
      }
#pragma unroll
      for (int o = 0; o < TH; ++o) {
        const int ti = ir - o;
        if (ti < 0 || ti >= KS) continue;
#pragma unroll
        for (int tj = 0; tj < KS; ++tj) acc[o] = fma2(xv[tj], wr[ti * KS + tj], acc[o]);
      }
    }
#pragma unroll
    for (int o = 0; o < TH; ++o) {
      const int h = h0 + o;
      if (h >= H) continue;
      float va, vb;
      upk2(acc[o], va, vb);
      if (gelu) gelu_tanh_x2(va, vb);
      *reinterpret_cast<uint32_t*>(y + (((size_t)n * H + h) * W + w0 + wl) * C + cs0 + 2 * cp) = float2_to_bf16x2(va, vb);
    }
  }
}

template <int KS, int CG, int NC, int TH>
static int launch_dwconv_tiled(const __nv_bfloat16* x, const float* wk, const float* bias, const float* pre_a,
                               const float* pre_b, __nv_bfloat16* y, int Nimg, int H, int W, int C,
                               int add_centre, int gelu, cudaStream_t st) {
  constexpr int TW = CG * NC;
  const size_t smem = (size_t)(TH + KS - 1) * (TW + KS - 1) * 64 * 2;
  cudaError_t e = cudaFuncSetAttribute(dwconv_tiled_kernel<KS, CG, NC, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const long long grid = (long long)Nimg * ((H + TH - 1) / TH) * ((W + TW - 1) / TW) * (C / 64);
  dwconv_tiled_kernel<KS, CG, NC, TH><<<(unsigned)grid, 32 * CG, smem, st>>>(x, wk, bias, pre_a, pre_b, y, H, W, C,
                                                                            add_centre, gelu);
  return check_launch();
}

int launch_dwconv_cl(const __nv_bfloat16* x, const float* wk, const float* bias, const float* pre_a,
                     const float* pre_b, __nv_bfloat16* y, float* y_f32, int Nimg, int H, int W, int C,
                     int ks, int add_centre, int gelu, cudaStream_t st) {
  if (C % 8 != 0 || (ks != 3 && ks != 7)) return CSSM_ERR_UNSUPPORTED;
  if (y_f32 == nullptr && C % 64 == 0 && (wk == nullptr || (aligned16(wk) && (bias == nullptr || aligned16(bias))))) {
#define CSSM_DW(KS_, CG_, NC_, TH_) \
  return launch_dwconv_tiled<KS_, CG_, NC_, TH_>(x, wk, bias, pre_a, pre_b, y, Nimg, H, W, C, add_centre, gelu, st)
    if (ks == 7) {
      if (W % 28 == 0 && H % 8 != 0 && H % 7 == 0) CSSM_DW(7, 4, 7, 7);      // 28 x 28 planes
      if (W % 28 == 0) CSSM_DW(7, 4, 7, 8);                                  // 56 x 56 planes
      CSSM_DW(7, 4, 4, 8);
    }
    if (W == 14 && H == 14) CSSM_DW(3, 2, 7, 7);                             // two tiles per plane
    if (W == 7 && H == 7) CSSM_DW(3, 1, 7, 7);
    CSSM_DW(3, 4, 4, 8);
#undef CSSM_DW
  }
  constexpr int RH = 4;
  const size_t smem = (size_t)(ks * ks * C + C) * 4;
  const long long total = (long long)Nimg * ((H + RH - 1) / RH) * W * (C / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaError_t e;
  if (ks == 3) {
    e = cudaFuncSetAttribute(dwconv_cl_kernel<3, RH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    dwconv_cl_kernel<3, RH><<<(int)blocks, 256, smem, st>>>(x, wk, bias, pre_a, pre_b, y, y_f32, Nimg, H, W, C,
                                                             add_centre, gelu);
  } else {
    e = cudaFuncSetAttribute(dwconv_cl_kernel<7, RH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
    dwconv_cl_kernel<7, RH><<<(int)blocks, 256, smem, st>>>(x, wk, bias, pre_a, pre_b, y, y_f32, Nimg, H, W, C,
                                                             add_centre, gelu);
  }
  return check_launch();
}

// ------------------------------------------------------------------ LayerNorm over C ----
// Per-pixel LayerNorm (eps 1e-6) on channels-last bf16.  A pixel is handled by C/8 consecutive
// threads (8 channels = 16 bytes each); partial sums meet in shared memory; two passes (mean,
// then squared deviations) on the values kept in registers.
__global__ void __launch_bounds__(256)
layernorm_cl_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                    const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, long long npix, int C,
                    int ppb) {
  __shared__ float part[256];
  __shared__ float stat[256];
  const int chunks = C / 8;
  const int lp = threadIdx.x / chunks, ck = threadIdx.x - lp * chunks;
  const long long px = (long long)blockIdx.x * ppb + lp;
  const bool on = lp < ppb && px < npix;
  float v[8];
  if (on) unpack8(__ldg(reinterpret_cast<const uint4*>(x + px * C + ck * 8)), v);
  else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += v[j];
  part[threadIdx.x] = s;
  __syncthreads();
  if (on && ck == 0) {
    float t = 0.f;
    for (int i = 0; i < chunks; ++i) t += part[lp * chunks + i];
    stat[lp] = t / (float)C;
  }
  __syncthreads();
  const float mean = on ? stat[lp] : 0.f;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { const float d = v[j] - mean; q = fmaf(d, d, q); }
  __syncthreads();
  part[threadIdx.x] = q;
  __syncthreads();
  if (on && ck == 0) {
    float t = 0.f;
    for (int i = 0; i < chunks; ++i) t += part[lp * chunks + i];
    stat[lp] = rsqrtf(t / (float)C + 1e-6f);
  }
  __syncthreads();
  if (!on) return;
  const float rstd = stat[lp];
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * __ldg(scale + ck * 8 + j) + __ldg(bias + ck * 8 + j);
  *reinterpret_cast<uint4*>(y + px * C + ck * 8) = pack8(o);
}
// The same for C / 8 a power of two of at most 32 lanes: the lanes of a pixel are a segment of one
// warp, so the two reductions are shuffles and the kernel needs no barrier.  A thread handles PP
// pixels (a grid-sized stride apart) and issues all their loads before it touches any: with one
// 16-byte load per thread the kernel ran at 0.61 of the copy bandwidth, bound by load latency.
// C = 8 G R: the G lanes of a pixel each own R 16-byte chunks (chunk = lane + r G), PP pixels per thread.
template <int G, int R, int PP>
__global__ void __launch_bounds__(256)
layernorm_cl_shfl_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                         const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, long long npix) {
  constexpr int C = G * R * 8;
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long pstride = (long long)gridDim.x * (256 / G);      // pixels covered by one pass of the grid
  const long long px0 = gid / G;
  const int ck = (int)(gid % G);
  uint4 raw[PP][R];
#pragma unroll
  for (int p = 0; p < PP; ++p) {
    const long long px = px0 + p * pstride;
#pragma unroll
    for (int r = 0; r < R; ++r)
      raw[p][r] = px < npix ? __ldg(reinterpret_cast<const uint4*>(x + px * C + (ck + r * G) * 8))
                            : make_uint4(0u, 0u, 0u, 0u);
  }
  // scale and bias of this lane's chunks, fetched alongside the pixels
  float sc[R][8], bi[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int c0 = (ck + r * G) * 8;
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(scale + c0)), s1 = __ldg(reinterpret_cast<const float4*>(scale + c0 + 4));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + c0)), b1 = __ldg(reinterpret_cast<const float4*>(bias + c0 + 4));
    sc[r][0] = s0.x; sc[r][1] = s0.y; sc[r][2] = s0.z; sc[r][3] = s0.w; sc[r][4] = s1.x; sc[r][5] = s1.y; sc[r][6] = s1.z; sc[r][7] = s1.w;
    bi[r][0] = b0.x; bi[r][1] = b0.y; bi[r][2] = b0.z; bi[r][3] = b0.w; bi[r][4] = b1.x; bi[r][5] = b1.y; bi[r][6] = b1.z; bi[r][7] = b1.w;
  }
#pragma unroll
  for (int p = 0; p < PP; ++p) {
    const long long px = px0 + p * pstride;
    float v[R][8];
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      unpack8(raw[p][r], v[r]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[r][j];
    }
#pragma unroll
    for (int o = G / 2; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * (1.0f / C);
    float q = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float d = v[r][j] - mean; q = fmaf(d, d, q); }
#pragma unroll
    for (int o = G / 2; o; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (px >= npix) continue;                      // after the shuffles: whole pixels are in or out
    const float rstd = rsqrtf(q * (1.0f / C) + 1e-6f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float o8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o8[j] = fmaf((v[r][j] - mean) * rstd, sc[r][j], bi[r][j]);
      *reinterpret_cast<uint4*>(y + px * C + (ck + r * G) * 8) = pack8(o8);
    }
  }
}
template <int G, int R, int PP>
static void launch_ln_shfl(const __nv_bfloat16* x, const float* scale, const float* bias, __nv_bfloat16* y,
                           long long npix, cudaStream_t st) {
  const long long blocks = (npix * G + 256 * PP - 1) / (256 * PP);
  layernorm_cl_shfl_kernel<G, R, PP><<<(unsigned)blocks, 256, 0, st>>>(x, scale, bias, y, npix);
}

int launch_layernorm_cl(const __nv_bfloat16* x, const float* scale, const float* bias, __nv_bfloat16* y,
                        long long npix, int C, cudaStream_t st) {
  if (C % 8 != 0 || C / 8 > 256) return CSSM_ERR_UNSUPPORTED;
  if (aligned16(scale) && aligned16(bias)) {
    switch (C) {
      case 32:  launch_ln_shfl<4, 1, 4>(x, scale, bias, y, npix, st); return check_launch();
      case 64:  launch_ln_shfl<8, 1, 4>(x, scale, bias, y, npix, st); return check_launch();
      case 128: launch_ln_shfl<16, 1, 4>(x, scale, bias, y, npix, st); return check_launch();
      case 256: launch_ln_shfl<32, 1, 4>(x, scale, bias, y, npix, st); return check_launch();
      case 384: launch_ln_shfl<16, 3, 2>(x, scale, bias, y, npix, st); return check_launch();
      case 512: launch_ln_shfl<32, 2, 2>(x, scale, bias, y, npix, st); return check_launch();
      default: break;
    }
  }
  const int chunks = C / 8, ppb = 256 / chunks;
  const long long blocks = (npix + ppb - 1) / ppb;
  layernorm_cl_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, scale, bias, y, npix, C, ppb);
  return check_launch();
}

// ------------------------------------------------------------------ LayerNorm over a sample ----
// Moments over all H*W*C values of each sample (two passes over the L2-resident sample), written as
// the per-(sample, channel) affine the consumer applies on load:
//   a[n, c] = rstd_n * scale[c],  b[n, c] = bias[c] - mean_n * rstd_n * scale[c].
__global__ void __launch_bounds__(512)
sample_norm_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                   const float* __restrict__ bias, float* __restrict__ a, float* __restrict__ b, int per,
                   int C) {
  __shared__ float red[16];
  __shared__ float bc;
  const int n = blockIdx.x;
  const uint4* xs = reinterpret_cast<const uint4*>(x + (size_t)n * per);
  const int chunks = per / 8;
  auto block_sum = [&](float s) {
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
      bc = t;
    }
    __syncthreads();
    return bc;
  };
  float s = 0.f;
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
    float v[8];
    unpack8(__ldg(xs + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j];
  }
  const float mean = block_sum(s) / (float)per;
  float q = 0.f;
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
    float v[8];
    unpack8(__ldg(xs + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float d = v[j] - mean; q = fmaf(d, d, q); }
  }
  const float rstd = rsqrtf(block_sum(q) / (float)per + 1e-6f);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float sc = rstd * scale[c];
    a[(size_t)n * C + c] = sc;
    b[(size_t)n * C + c] = bias[c] - mean * sc;
  }
}
int launch_sample_norm(const __nv_bfloat16* x, const float* scale, const float* bias, float* a, float* b,
                       int Nimg, int per, int C, cudaStream_t st) {
  if (per % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  sample_norm_kernel<<<Nimg, 512, 0, st>>>(x, scale, bias, a, b, per, C);
  return check_launch();
}

// ------------------------------------------------------------------ plane sums ----
// sums[n, c] = sum over the P pixels of x[n, p, c] (x has row stride ld): thread = 8 channels of a
// slice of the pixels; deterministic order.
__global__ void __launch_bounds__(256)
plane_sum_cl_kernel(const __nv_bfloat16* __restrict__ x, int ld, int P, int C, float* __restrict__ sums) {
  __shared__ float part[8][33][8];
  const int chunks = C / 8;                          // blockDim.x = 32 chunk lanes, blockDim.y = 8 pixel slices
  const int n = blockIdx.y, ck = blockIdx.x * 32 + threadIdx.x;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (ck < chunks) {
    const __nv_bfloat16* xp = x + (size_t)n * P * ld + ck * 8;
    for (int p = threadIdx.y; p < P; p += 8) {
      float v[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(xp + (size_t)p * ld)), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && ck < chunks) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.f;
      for (int s = 0; s < 8; ++s) t += part[s][threadIdx.x][j];
      sums[(size_t)n * C + ck * 8 + j] = t;
    }
  }
}
int launch_plane_sum_cl(const __nv_bfloat16* x, int ld, int Nimg, int P, int C, float* sums, cudaStream_t st) {
  if (C % 8 != 0 || ld % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  dim3 grid((C / 8 + 31) / 32, Nimg), block(32, 8);
  plane_sum_cl_kernel<<<grid, block, 0, st>>>(x, ld, P, C, sums);
  return check_launch();
}

// ------------------------------------------------------------------ readout ----
// pooled[n, c] = max (or mean) over the P pixels of x[n, p, c], float32.
__global__ void pool_cl_kernel(const __nv_bfloat16* __restrict__ x, int P, int C, int use_max,
                               float* __restrict__ pooled) {
  const int n = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const __nv_bfloat16* xp = x + (size_t)n * P * C + c;
  float m = use_max ? -INFINITY : 0.f;
  for (int p = 0; p < P; ++p) {
    const float v = __bfloat162float(xp[(size_t)p * C]);
    m = use_max ? fmaxf(m, v) : m + v;
  }
  pooled[(size_t)n * C + c] = use_max ? m : m / (float)P;
}
int launch_pool_cl(const __nv_bfloat16* x, int Nimg, int P, int C, int use_max, float* pooled, cudaStream_t st) {
  dim3 grid((C + 127) / 128, Nimg);
  pool_cl_kernel<<<grid, 128, 0, st>>>(x, P, C, use_max, pooled);
  return check_launch();
}

// logits[n, k] = pooled[n, :] . W[:, k] + b[k], float32 (the reference keeps its head in float32).
// A CTA computes 128 classes for 8 samples, so a weight read feeds eight accumulators.
__global__ void __launch_bounds__(128)
head_kernel(const float* __restrict__ pooled, const float* __restrict__ W, const float* __restrict__ b,
            float* __restrict__ logits, int Nimg, int C, int K) {
  extern __shared__ __align__(16) float ps[];        // [8][C], C a multiple of 4 for the float4 reads
  const int n0 = blockIdx.y * 8;
  for (int i = threadIdx.x; i < 8 * C; i += blockDim.x) {
    const int j = i / C, c = i - j * C;
    ps[i] = n0 + j < Nimg ? pooled[(size_t)(n0 + j) * C + c] : 0.f;
  }
  __syncthreads();
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = b[k];
  // eight weight loads in flight per thread; the pooled values are read as float4 (one shared-memory
  // load per four channels: the loop is bound by the number of shared-memory instructions otherwise)
  int c = 0;
  for (; c + 8 <= C; c += 8) {
    float w[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) w[u] = __ldg(W + (size_t)(c + u) * K + k);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 p0 = *reinterpret_cast<const float4*>(ps + j * C + c);
      const float4 p1 = *reinterpret_cast<const float4*>(ps + j * C + c + 4);
      acc[j] = fmaf(p0.x, w[0], acc[j]); acc[j] = fmaf(p0.y, w[1], acc[j]);
      acc[j] = fmaf(p0.z, w[2], acc[j]); acc[j] = fmaf(p0.w, w[3], acc[j]);
      acc[j] = fmaf(p1.x, w[4], acc[j]); acc[j] = fmaf(p1.y, w[5], acc[j]);
      acc[j] = fmaf(p1.z, w[6], acc[j]); acc[j] = fmaf(p1.w, w[7], acc[j]);
    }
  }
  for (; c < C; ++c) {
    const float w = __ldg(W + (size_t)c * K + k);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = fmaf(ps[j * C + c], w, acc[j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (n0 + j < Nimg) logits[(size_t)(n0 + j) * K + k] = acc[j];
}
// The same product with the weights read from L2 once per CTA instead of once per eight samples: a CTA
// keeps a slice of 64 classes (C x 64 floats) and its share of the pooled rows in shared memory, about
// one CTA per SM; thread = one class x every fourth sample of the CTA, four samples at a time.
constexpr int HT_K = 64;
__global__ void __launch_bounds__(256)
head_tile_kernel(const float* __restrict__ pooled, const float* __restrict__ W, const float* __restrict__ b,
                 float* __restrict__ logits, int Nimg, int C, int K, int spc) {
  extern __shared__ __align__(16) float hs[];
  float* Ws = hs;                                      // [C][64]
  float* ps = hs + (size_t)C * HT_K;                   // [spc][C]
  const int k0 = blockIdx.x * HT_K, n0 = blockIdx.y * spc;
  const int ns = Nimg - n0 < spc ? Nimg - n0 : spc;
  for (int i = threadIdx.x; i < C * (HT_K / 4); i += 256) {
    const int c = i / (HT_K / 4), k4 = (i - c * (HT_K / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k0 + k4 < K) v = __ldg(reinterpret_cast<const float4*>(W + (size_t)c * K + k0 + k4));   // K % 4 == 0
    *reinterpret_cast<float4*>(Ws + c * HT_K + k4) = v;
  }
  for (int i = threadIdx.x; i < ns * (C / 4); i += 256)
    reinterpret_cast<float4*>(ps)[i] = __ldg(reinterpret_cast<const float4*>(pooled + (size_t)n0 * C) + i);
  __syncthreads();
  const int kk = threadIdx.x & (HT_K - 1), sl = threadIdx.x / HT_K;      // class, sample lane 0..3
  if (k0 + kk >= K) return;
  const float bias = b[k0 + kk];
  for (int j0 = sl; j0 < ns; j0 += 16) {
    float acc[4] = {bias, bias, bias, bias};
    const float* pj[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) pj[m] = ps + (size_t)(j0 + 4 * m < ns ? j0 + 4 * m : j0) * C;
    for (int c = 0; c < C; c += 4) {
      const float w0 = Ws[c * HT_K + kk], w1 = Ws[(c + 1) * HT_K + kk], w2 = Ws[(c + 2) * HT_K + kk],
                  w3 = Ws[(c + 3) * HT_K + kk];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float4 p = *reinterpret_cast<const float4*>(pj[m] + c);
        acc[m] = fmaf(p.x, w0, acc[m]); acc[m] = fmaf(p.y, w1, acc[m]);
        acc[m] = fmaf(p.z, w2, acc[m]); acc[m] = fmaf(p.w, w3, acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m)
      if (j0 + 4 * m < ns) logits[(size_t)(n0 + j0 + 4 * m) * K + k0 + kk] = acc[m];
  }
}
int launch_head(const float* pooled, const float* W, const float* b, float* logits, int Nimg, int C, int K,
                cudaStream_t st) {
  if (C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (K % 4 == 0 && Nimg >= 64 && aligned16(W) && aligned16(pooled)) {
    const int nx = (K + HT_K - 1) / HT_K;
    int ny = 148 / nx > 0 ? 148 / nx : 1;
    int spc = (Nimg + ny - 1) / ny;
    const size_t cap = 200 * 1024;
    const size_t wbytes = (size_t)C * HT_K * 4;
    if (wbytes + 4 * (size_t)C * 4 <= cap) {
      const int spc_max = (int)((cap - wbytes) / ((size_t)C * 4));
      if (spc > spc_max) spc = spc_max;
      ny = (Nimg + spc - 1) / spc;
      const size_t smem = wbytes + (size_t)spc * C * 4;
      cudaError_t e = cudaFuncSetAttribute(head_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
      head_tile_kernel<<<dim3(nx, ny), 256, smem, st>>>(pooled, W, b, logits, Nimg, C, K, spc);
      return check_launch();
    }
  }
  dim3 grid((K + 127) / 128, (Nimg + 7) / 8);
  head_kernel<<<grid, 128, (size_t)8 * C * 4, st>>>(pooled, W, b, logits, Nimg, C, K);
  return check_launch();
}

// ------------------------------------------------------------------ conversions ----
__global__ void f32_to_bf16_vec_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * i), b = __ldg(reinterpret_cast<const float4*>(x) + 2 * i + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    reinterpret_cast<uint4*>(y)[i] = pack8(v);
  }
}
int launch_f32_to_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t st) {
  if (n % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  f32_to_bf16_vec_kernel<<<(int)blocks, 256, 0, st>>>(x, y, n / 8);
  return check_launch();
}

// out = res + y (res bf16, y float32) -> bf16: the residual after the general (float32) mixer path
__global__ void add_res_kernel(const __nv_bfloat16* __restrict__ res, const float* __restrict__ yv,
                               __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float r[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(res) + i), r);
    const float4 a = __ldg(reinterpret_cast<const float4*>(yv) + 2 * i), b = __ldg(reinterpret_cast<const float4*>(yv) + 2 * i + 1);
    r[0] += a.x; r[1] += a.y; r[2] += a.z; r[3] += a.w; r[4] += b.x; r[5] += b.y; r[6] += b.z; r[7] += b.w;
    reinterpret_cast<uint4*>(out)[i] = pack8(r);
  }
}
int launch_add_res(const __nv_bfloat16* res, const float* yv, __nv_bfloat16* out, long long n, cudaStream_t st) {
  if (n % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  add_res_kernel<<<(int)blocks, 256, 0, st>>>(res, yv, out, n / 8);
  return check_launch();
}

}  // namespace cssm
