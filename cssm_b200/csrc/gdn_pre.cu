// GDN block, kernels ahead of the spectral stage: RoPE + channels-last depthwise conv with
// per-row context sums, and the gate maps (alpha, beta per frequency bin; B_k, B_v per pixel).
#include "kernels.cuh"
#include "bf16_ops.cuh"

namespace cssm {

// ------------------------------------------------- RoPE + depthwise KxK, channels-last ----
// One CTA per (frame, band of DW_ROWS output rows, group of 16 channels).  The band's input
// rows (+ halo) are rotated (RoPE) while they are staged in shared memory as [row][w][16];
// each thread then produces DW_ROWS x 4 outputs for one channel from there.  The CTA also
// writes, per centre row and channel, the sum over w of the ROTATED INPUT (ctx is the mean of
// the block input, cssm.py:4785-4786), not of the conv output.
constexpr int DW_ROWS = 8, DW_THREADS = 256;

// Position of (padded column col, channel c) inside a staged row.  With 16 channels per pixel two
// pixels share a 32-float line; the halves swap with bit 2 of the column, so that the two
// half-warps of a window read (columns col and col + 4, same channels) hit different banks.
template <int DW_CG>
__device__ __forceinline__ int dw_pos(int col, int c) {
  if (DW_CG == 16) return ((col >> 1) << 5) + ((((col & 1) ^ ((col >> 2) & 1))) << 4) + c;
  return col * DW_CG + c;
}

template <int K, int DW_CG>
__global__ void __launch_bounds__(DW_THREADS, (K <= 5 ? 2 : 1)) rope_dwconv_cl_kernel(const GdnDwArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int LO = (K - 1) / 2, NR = DW_ROWS + K - 1;
  const int W = a.W, C = a.C, n2 = C / 2;
  const int WP = (W + K - 1 + 1) & ~1;                 // padded columns per staged row (even)
  const int rpitch = WP * DW_CG;                        // floats per staged row
  const int bands = (a.H + DW_ROWS - 1) / DW_ROWS, cgs = C / DW_CG;
  int bid = blockIdx.x;
  const int cg = bid % cgs; bid /= cgs;
  const int band = bid % bands;
  const int fr = bid / bands;
  const int t = fr % a.T, h0 = band * DW_ROWS, c0 = cg * DW_CG;
  const int fsrc = a.x_bcast ? fr / a.T : fr;
  const int tid = threadIdx.x;
  // ---- zero the pad columns (left LO, right up to WP) of every staged row ----
  for (int i = tid; i < NR * (WP - W) * DW_CG; i += DW_THREADS) {
    const int r = i / ((WP - W) * DW_CG), rem = i - r * (WP - W) * DW_CG;
    const int pc = rem / DW_CG, c = rem - pc * DW_CG;
    const int col = pc < LO ? pc : W + pc;               // 0..LO-1, then W+LO..WP-1
    sm[r * rpitch + dw_pos<DW_CG>(col, c)] = 0.f;
  }
  // ---- stage rows h0-LO .. h0+DW_ROWS-1+(K-1-LO), DW_CG channels, rotated ----
  // DW_THREADS is a multiple of the pairs per pixel, so a thread keeps its channel pair and walks
  // columns wb, wb + WSTEP of every staged row: the t part of the angle is loaded once, the w part
  // once per column, the h part once per row.  Four rows x two columns are fetched per trip, every
  // load issued before the first is used.
  constexpr int PP = DW_CG / 2;                         // pairs per pixel in this channel group
  constexpr int WSTEP = DW_THREADS / PP;
  const int pl = tid % PP, pi = c0 / 2 + pl;
  const bool rope = a.rope_t != nullptr;
  float2 ct = make_float2(1.f, 0.f);
  if (rope) ct = a.rope_t[t * n2 + pi];
  const float* xf = a.x + (size_t)fsrc * a.H * W * C + c0 + 2 * pl;
  for (int wb = tid / PP; wb < W; wb += 2 * WSTEP) {
    float2 cw[2];
    int spos[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int w = wb + k * WSTEP;
      cw[k] = (rope && w < W) ? __ldg(&a.rope_w[w * n2 + pi]) : make_float2(1.f, 0.f);
      spos[k] = dw_pos<DW_CG>(min(w, W - 1) + LO, 2 * pl);
    }
#pragma unroll
    for (int r0 = 0; r0 < NR; r0 += 4) {
      float2 v[4][2];
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int hh = h0 + r0 + r4 - LO;
        const bool rin = r0 + r4 < NR && hh >= 0 && hh < a.H;
#pragma unroll
        for (int k = 0; k < 2; ++k)
          v[r4][k] = (rin && wb + k * WSTEP < W)
                         ? __ldg(reinterpret_cast<const float2*>(xf + ((size_t)hh * W + wb + k * WSTEP) * C))
                         : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        if (r0 + r4 >= NR) continue;
        const int hh = h0 + r0 + r4 - LO;
        float cth = 1.f, sth = 0.f;
        if (rope && hh >= 0 && hh < a.H) {
          const float2 ch = __ldg(&a.rope_h[hh * n2 + pi]);
          cth = ct.x * ch.x - ct.y * ch.y; sth = ct.x * ch.y + ct.y * ch.x;
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (wb + k * WSTEP >= W) continue;
          const float c2 = cth * cw[k].x - sth * cw[k].y, s2 = cth * cw[k].y + sth * cw[k].x;
          const float2 o = make_float2(v[r4][k].x * c2 - v[r4][k].y * s2, v[r4][k].x * s2 + v[r4][k].y * c2);
          *reinterpret_cast<float2*>(sm + (r0 + r4) * rpitch + spos[k]) = o;
        }
      }
    }
  }
  __syncthreads();
  // ---- context partial sums of the centre rows ----
  if (a.ctx_part != nullptr && tid < DW_ROWS * DW_CG) {
    const int r = tid / DW_CG, c = tid % DW_CG;
    if (h0 + r < a.H) {
      float s = 0.f;
      const float* srow = sm + (r + LO) * rpitch;
      for (int w = 0; w < W; ++w) s += srow[dw_pos<DW_CG>(w + LO, c)];
      a.ctx_part[((size_t)fr * a.H + h0 + r) * C + c0 + c] = s;
    }
  }
  if (a.out == nullptr) return;
  // ---- conv: thread = (channel pair, two consecutive w), all DW_ROWS rows; packed f32x2 FMAs ----
  // The staged pairs are read with 8-byte loads as they lie.  With eight pairs per pixel a warp holds
  // four column pairs; they are taken in the order 0, 2, 1, 3 so that the two of a half-warp are four
  // columns apart and land in different halves of the swizzled 128-byte lines.
  unsigned long long wk2[K * K];
#pragma unroll
  for (int i = 0; i < K * K; ++i) {
    const float2 w2 = *reinterpret_cast<const float2*>(a.wk + (size_t)i * C + c0 + 2 * pl);
    wk2[i] = pk2(w2.x, w2.y);
  }
  const float2 b2 = *reinterpret_cast<const float2*>(a.bias + c0 + 2 * pl);
  const unsigned long long bias2 = pk2(b2.x, b2.y);
  const int q = tid / PP;
  const int qs = PP == 8 ? ((q & ~3) | ((q & 1) << 1) | ((q >> 1) & 1)) : q;
  for (int wg = qs; wg * 2 < W; wg += WSTEP) {
    const int w0 = wg * 2;
    unsigned long long acc[DW_ROWS][2];
#pragma unroll
    for (int r = 0; r < DW_ROWS; ++r) { acc[r][0] = bias2; acc[r][1] = bias2; }
    // offsets of the window's padded columns w0 .. w0+K inside a staged row (same for all rows)
    int off[2 + K - 1];
#pragma unroll
    for (int j = 0; j < 2 + K - 1; ++j) off[j] = dw_pos<DW_CG>(min(w0 + j, WP - 1), 2 * pl);
#pragma unroll
    for (int ir = 0; ir < NR; ++ir) {
      const float* srow = sm + ir * rpitch;
      unsigned long long win[2 + K - 1];
#pragma unroll
      for (int j = 0; j < 2 + K - 1; ++j)
        win[j] = *reinterpret_cast<const unsigned long long*>(srow + off[j]);   // pad columns hold zeros
      // input row ir feeds output row r = ir - di for tap row di
#pragma unroll
      for (int di = 0; di < K; ++di) {
        const int r = ir - di;
        if (r < 0 || r >= DW_ROWS) continue;
#pragma unroll
        for (int dj = 0; dj < K; ++dj) {
          acc[r][0] = fma2(wk2[di * K + dj], win[dj], acc[r][0]);
          acc[r][1] = fma2(wk2[di * K + dj], win[dj + 1], acc[r][1]);
        }
      }
    }
    float* orow = a.out + (((size_t)fr * a.H + h0) * W + w0) * C + c0 + 2 * pl;
#pragma unroll
    for (int r = 0; r < DW_ROWS; ++r) {
      if (h0 + r >= a.H) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (w0 + j < W) {
          float ox, oy;
          upk2(acc[r][j], ox, oy);
          *reinterpret_cast<float2*>(orow + ((size_t)r * W + j) * C) = make_float2(ox, oy);
        }
    }
  }
}

// ------------------------------------------- context row sums without a conv (K = 1) ----
// ctx_part[(frame, h, c)] = sum over w of the rotated input.  One warp per image row: a lane
// owns channel pairs lane, lane + 32, ... and walks the row, so every load is a coalesced
// C*4-byte line and no cross-lane reduction is needed.  The t and h parts of the angle are
// combined once per row, the w part comes from the table per element.
constexpr int CTX_WARPS = 8;
__global__ void __launch_bounds__(CTX_WARPS * 32) rope_ctx_rowsum_kernel(const GdnDwArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * CTX_WARPS + warp;        // (frame, h)
  if (row >= (long long)a.BT * a.H) return;
  const int fr = (int)(row / a.H), h = (int)(row % a.H);
  const int t = fr % a.T, n2 = a.C / 2;
  const int fsrc = a.x_bcast ? fr / a.T : fr;
  const float* xr = a.x + ((size_t)fsrc * a.H + h) * a.W * a.C;
  for (int pi = lane; pi < n2; pi += 32) {
    float cth = 1.f, sth = 0.f;
    if (a.rope_t != nullptr) {
      const float2 ct = a.rope_t[t * n2 + pi], ch = a.rope_h[h * n2 + pi];
      cth = ct.x * ch.x - ct.y * ch.y; sth = ct.x * ch.y + ct.y * ch.x;
    }
    float se = 0.f, so = 0.f;
#pragma unroll 4
    for (int w = 0; w < a.W; ++w) {
      const float2 v = __ldg(reinterpret_cast<const float2*>(xr + (size_t)w * a.C + 2 * pi));
      if (a.rope_t != nullptr) {
        const float2 cw = __ldg(&a.rope_w[w * n2 + pi]);
        const float c2 = cth * cw.x - sth * cw.y, s2 = cth * cw.y + sth * cw.x;
        se += v.x * c2 - v.y * s2; so += v.x * s2 + v.y * c2;
      } else {
        se += v.x; so += v.y;
      }
    }
    *reinterpret_cast<float2*>(a.ctx_part + (size_t)row * a.C + 2 * pi) = make_float2(se, so);
  }
}

template <int K, int DW_CG>
static int launch_dw_cg(const GdnDwArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)(DW_ROWS + K - 1) * ((a.W + K - 1 + 1) & ~1) * DW_CG * sizeof(float);
  if (smem > 200 * 1024) return CSSM_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(rope_dwconv_cl_kernel<K, DW_CG>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const int bands = (a.H + DW_ROWS - 1) / DW_ROWS;
  rope_dwconv_cl_kernel<K, DW_CG><<<a.BT * bands * (a.C / DW_CG), DW_THREADS, smem, st>>>(a);
  return check_launch();
}

// 16-channel groups (64-byte segments per pixel) when C allows, else 4-channel groups
template <int K>
static int launch_dw(const GdnDwArgs& a, cudaStream_t st) {
  return a.C % 16 == 0 ? launch_dw_cg<K, 16>(a, st) : launch_dw_cg<K, 4>(a, st);
}

int launch_rope_dwconv_cl(const GdnDwArgs& a, cudaStream_t st) {
  if (a.C % 4 != 0) return CSSM_ERR_UNSUPPORTED;
  if (a.ksz <= 1 && a.out == nullptr) {
    if (a.ctx_part == nullptr) return CSSM_OK;
    const long long rows = (long long)a.BT * a.H;
    rope_ctx_rowsum_kernel<<<(unsigned)((rows + CTX_WARPS - 1) / CTX_WARPS), CTX_WARPS * 32, 0, st>>>(a);
    return check_launch();
  }
  switch (a.ksz > 1 ? a.ksz : 1) {
    case 1: return launch_dw<1>(a, st);
    case 3: return launch_dw<3>(a, st);
    case 5: return launch_dw<5>(a, st);
    case 7: return launch_dw<7>(a, st);
    default: return CSSM_ERR_UNSUPPORTED;
  }
}

// ------------------------------------------------------------------- GDN gate maps ----
// One CTA per frame.  ctx = (sum over rows of ctx_part) / (H*W) + tcode[t].
// alpha/beta: sigmoid(row[h] + col[kw]) (factored) or sigmoid(Dense(H*Wf)) (dense);
// alpha = 0.1 + 0.89 * raw.  Stored as float2 {alpha, beta} at bin_index(path, kh, kw).
// B_k / B_v: same over (h, w) pixels, float2 {B_k, B_v} at h*W + w.  cssm.py:4798-4848, 4864-4865.
__global__ void __launch_bounds__(256) gdn_gates_kernel(const GdnGateArgs g) {
  extern __shared__ float sh[];
  const int Wf = g.W / 2 + 1, NB = g.H * Wf, HW = g.H * g.W;
  float* ctx = sh;                       // [C]
  float* vec = sh + g.C;                 // factored: alpha_h, alpha_w, beta_h, beta_w, Bk_h, Bk_w, Bv_h, Bv_w
  const int fr = blockIdx.x, tid = threadIdx.x, t = fr % g.T;
  const float inv = 1.0f / (float)HW;
  for (int c = tid; c < g.C; c += blockDim.x) {
    float s = 0.f;
    const int fsrc = g.ctx_per_clip ? fr / g.T : fr;
    for (int h = 0; h < g.H; ++h) s += g.ctx_part[((size_t)fsrc * g.H + h) * g.C + c];
    ctx[c] = s * inv + g.tcode[t * g.C + c];
  }
  __syncthreads();
  const int ngate = g.use_input_gates ? 4 : 2;
  if (g.gate_type == CSSM_GATE_FACTORED) {
    // segment offsets inside vec
    int off[9];
    off[0] = 0;
    for (int q = 0; q < 4; ++q) {
      const int wd = q < 2 ? Wf : g.W;
      off[2 * q + 1] = off[2 * q] + g.H;
      off[2 * q + 2] = off[2 * q + 1] + wd;
    }
    const int total = off[2 * ngate];
    for (int o = tid; o < total; o += blockDim.x) {
      int seg = 0;
      while (o >= off[seg + 1]) ++seg;
      const int col = o - off[seg];
      const int ncol = off[seg + 1] - off[seg];
      const float* kk = g.gk[seg];
      float acc = g.gb[seg][col];
      for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], kk[(size_t)c * ncol + col], acc);
      vec[o] = acc;
    }
    __syncthreads();
    for (int bin = tid; bin < NB; bin += blockDim.x) {
      const int kh = bin / Wf, kw = bin % Wf;
      const float ra = sigmoid_f(vec[off[0] + kh] + vec[off[1] + kw]);
      const float rb = sigmoid_f(vec[off[2] + kh] + vec[off[3] + kw]);
      g.ab[(size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf)] = make_float2(0.1f + 0.89f * ra, rb);
    }
    if (g.use_input_gates)
      for (int px = tid; px < HW; px += blockDim.x) {
        const int h = px / g.W, w = px % g.W;
        g.bkv[(size_t)fr * HW + px] = make_float2(sigmoid_f(vec[off[4] + h] + vec[off[5] + w]),
                                                  sigmoid_f(vec[off[6] + h] + vec[off[7] + w]));
      }
  } else if (g.gate_type == CSSM_GATE_SCALAR || g.gate_type == CSSM_GATE_CHANNEL) {
    // scalar: one value per frame and gate, Dense(1)(ctx) (cssm.py:4825-4833).  channel: alpha, beta
    // per head, Dense(n_h)(ctx) (cssm.py:4808-4810); its spatial gates are a 1x1 conv of the block
    // input and are applied elsewhere.  The maps are constant over the bins.
    const bool chan = g.gate_type == CSSM_GATE_CHANNEL;
    const int nout = chan ? g.nh : 1, nvec = chan ? 2 : ngate;
    for (int o = tid; o < nvec * nout; o += blockDim.x) {
      const int gi = o / nout, col = o - gi * nout;
      float acc = g.gb[gi][col];
      for (int c = 0; c < g.C; ++c) acc = fmaf(ctx[c], g.gk[gi][(size_t)c * nout + col], acc);
      vec[o] = sigmoid_f(acc);
    }
    __syncthreads();
    for (int i = tid; i < nout * NB; i += blockDim.x) {
      const int hh = i / NB;
      g.ab[((size_t)fr * nout + hh) * NB + (i - hh * NB)] = make_float2(0.1f + 0.89f * vec[hh], vec[nout + hh]);
    }
    if (!chan && g.use_input_gates)
      for (int px = tid; px < HW; px += blockDim.x) g.bkv[(size_t)fr * HW + px] = make_float2(vec[2], vec[3]);
  } else {
    for (int bin = tid; bin < NB; bin += blockDim.x) {
      const int kh = bin / Wf, kw = bin % Wf;
      float aa = g.gb[0][bin], bb = g.gb[1][bin];
      for (int c = 0; c < g.C; ++c) {
        aa = fmaf(ctx[c], g.gk[0][(size_t)c * NB + bin], aa);
        bb = fmaf(ctx[c], g.gk[1][(size_t)c * NB + bin], bb);
      }
      g.ab[(size_t)fr * NB + bin_index(g.path, kh, kw, g.H, Wf)] =
          make_float2(0.1f + 0.89f * sigmoid_f(aa), sigmoid_f(bb));
    }
    if (g.use_input_gates)
      for (int px = tid; px < HW; px += blockDim.x) {
        float aa = g.gb[2][px], bb = g.gb[3][px];
        for (int c = 0; c < g.C; ++c) {
          aa = fmaf(ctx[c], g.gk[2][(size_t)c * HW + px], aa);
          bb = fmaf(ctx[c], g.gk[3][(size_t)c * HW + px], bb);
        }
        g.bkv[(size_t)fr * HW + px] = make_float2(sigmoid_f(aa), sigmoid_f(bb));
      }
  }
}

int launch_gdn_gates(const GdnGateArgs& g, cudaStream_t st) {
  const size_t smem = (size_t)(g.C + 4 * g.H + 2 * (g.W / 2 + 1) + 2 * g.W + 2 * g.nh + 8) * sizeof(float);
  gdn_gates_kernel<<<g.BT, 256, smem, st>>>(g);
  return check_launch();
}

}  // namespace cssm
