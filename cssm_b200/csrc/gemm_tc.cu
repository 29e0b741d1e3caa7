// tcgen05 / TMEM GEMM for the K = 64 channel projections in fp32-equivalent precision
// (3 x TF32: A_hi*B_hi + A_lo*B_hi + A_hi*B_lo, accumulated in fp32 in TMEM).
//
// Persistent kernel, one CTA per SM, 544 threads, warp-specialised:
//   warps 0-7  producers : read a 128-pixel A tile from global memory (channels-last rows with
//                          RoPE fused, loaded one tile ahead into registers so a whole tile is
//                          in flight per SM; or planar planes with the RMSNorm/gate prologue
//                          fused), split every value into tf32 hi + remainder, and
//                          write both into the 128-byte-swizzled K-major operand layout of a
//                          2-stage ring;
//   warp  8    MMA issuer: one lane issues 24 tcgen05.mma (M128 x N x K8) per tile into one of
//                          two TMEM accumulators and commits to mbarriers;
//   warps 9-16 epilogue  : tcgen05.ld the accumulator (lane = pixel; two warps per TMEM lane
//                          quadrant, half of the columns each), add bias / activation, store
//                          planar (coalesced over pixels) or channels-last rows.
// The weight tile (both halves of the split) is prepared once per CTA and stays in shared memory.
// Every mbarrier wait is bounded; on expiry the kernel records an error code and winds down.
#include <cuda.h>
#include <string.h>
#include "kernels.cuh"
#include "gemm_simt.cuh"
#include "tc05.cuh"

namespace cssm {

__device__ int g_tc_error = 0;

constexpr int TC_THREADS = 544;      // 8 producer warps, 1 MMA warp, 8 epilogue warps
constexpr int TC_MMA_WARP = 8;
constexpr int TC_BM = 128;
constexpr int TC_K = 64;
constexpr uint32_t TC_A_HALF = 2u * TC_BM * 128u;      // one of hi / lo: 2 K-blocks x 128 rows x 128 B

// STG = false: the epilogue warps store straight from registers.
// STG = true : the epilogue stages 16 KB chunks (128 pixels x 32 output columns) in shared memory,
//              one chunk buffer per half of the epilogue warps, and writes each chunk with one TMA
//              tensor store (N <= 128: two A stages + two chunk buffers fit in 227 KB).
template <int N, bool STG>
struct TcSmem {
  static constexpr uint32_t NSTAGE = 2u;
  static constexpr uint32_t B_HALF = 2u * N * 128u;
  static constexpr uint32_t B_OFF = 0;
  static constexpr uint32_t A_OFF = 2u * B_HALF;                 // after B_hi, B_lo
  static constexpr uint32_t OUT_OFF = A_OFF + NSTAGE * 2u * TC_A_HALF;   // 2 x 16 KB when STG
  static constexpr uint32_t BIAS_OFF = OUT_OFF + (STG ? 2u * 16384u : 0u);
  static constexpr uint32_t BAR_OFF = BIAS_OFF + N * 4u;
  static constexpr uint32_t TOTAL = BAR_OFF + 128u;
};

// ZLAST: the output columns from act_n0 on (the z half of the in_proj) are only produced for the
// last frame of every clip (last-frame-only forward); a compile-time variant so that the default
// kernel carries no extra test.
template <int N, bool A_PLANAR, bool STG, bool ZLAST = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const GemmArgs g, int num_tiles, const __grid_constant__ CUtensorMap omap) {
  // tile schedule: round-robin over the CTAs
  const int t_first = blockIdx.x, t_step = gridDim.x, t_end = num_tiles;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // operand tiles need 1024-byte alignment (swizzle atoms); the launch adds 1024 bytes of slack
  unsigned char* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
  using L = TcSmem<N, STG>;
  constexpr int NSTAGE = L::NSTAGE;
  const uint32_t sbase = tc::smem_u32(smem);
  float* bias_s = reinterpret_cast<float*>(smem + L::BIAS_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* full = bars;          // [2] A stage written (128 producer arrivals)
  uint64_t* empty = bars + 2;     // [2] A stage consumed (tcgen05.commit)
  uint64_t* accfull = bars + 4;   // [2] accumulator complete (tcgen05.commit)
  uint64_t* accempty = bars + 6;  // [2] accumulator drained (128 epilogue arrivals)
  uint64_t* done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int NPROD = 256;                        // producer threads that arrive on `full`
  constexpr uint32_t TMEM_COLS = (2 * N <= 32) ? 32 : (2 * N <= 64) ? 64 : (2 * N <= 128) ? 128
                                 : (2 * N <= 256) ? 256 : 512;

  if (tid == 0) {
    tc::mbar_init(&full[0], NPROD / 32); tc::mbar_init(&full[1], NPROD / 32);      // one lane per producer warp
    tc::mbar_init(&empty[0], 1); tc::mbar_init(&empty[1], 1);
    tc::mbar_init(&accfull[0], 1); tc::mbar_init(&accfull[1], 1);
    tc::mbar_init(&accempty[0], 8); tc::mbar_init(&accempty[1], 8);                  // one lane per epilogue warp
    tc::mbar_init(done, 1);
    tc::fence_mbar_init();
  }
  if (warp == TC_MMA_WARP) {
    tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tmem_relinquish();
  }
  // ---- weights: W[k][n] -> B_hi / B_lo rows n, K-major swizzled ----
  for (int item = tid; item < N * 16; item += TC_THREADS) {
    const int n = item % N, c = item / N;               // c: 16-byte chunk of 4 k values
    float hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) tc::split_tf32(g.Wk[(size_t)(4 * c + e) * g.N + n], hi[e], lo[e]);
    const uint32_t off = (uint32_t)(c >> 3) * (N * 128u) + tc::sw128_offset(n, c & 7);
    *reinterpret_cast<float4*>(smem + L::B_OFF + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<float4*>(smem + L::B_OFF + L::B_HALF + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
  }
  for (int n = tid; n < N; n += TC_THREADS) bias_s[n] = g.bias ? g.bias[n] : 0.f;
  tc::fence_proxy_async();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8 && tid < NPROD) {
    // ================================ producers ================================
    int it = 0;
    // channels-last mode: the 128 x 16 float4 chunks of a tile are walked in two halves of four
    // iterations: iteration r covers chunk (tid & 7) + 8*(r >> 2) of row (tid >> 3) + 32*(r & 3),
    // so a warp load touches four rows x 128 contiguous bytes.  RoPE only rotates the low channel
    // pairs in most modes: a lane rotates in the half whose chunk holds a rotated pair, which
    // spreads the rotation evenly over all eight warps.  `pre` always holds the NEXT tile.
    float4 pre[8];
    const int chunk_lo = tid & 7, rsub = tid >> 3;
    bool rot[2] = {false, false};
    if (!A_PLANAR) {
      // a tile never crosses a frame (H*W is a multiple of the tile height), so the source-frame
      // remap is one row offset per tile
      const int m0 = t_first * TC_BM;
      const float* a0 = g.A + gemm_src_row(g, m0 < g.M ? m0 : 0) * TC_K;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int row = rsub + 32 * (r & 3);
        const int chunk = chunk_lo + 8 * (r >> 2);
        pre[r] = (t_first < t_end && m0 + row < g.M)
                     ? __ldg(reinterpret_cast<const float4*>(a0 + (size_t)row * TC_K + chunk * 4))
                     : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (g.rope_t != nullptr) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int pi = 2 * (chunk_lo + 8 * hf);
          rot[hf] = g.rope_nz == nullptr || g.rope_nz[pi] != 0.f || g.rope_nz[pi + 1] != 0.f;
        }
      }
    }
    const float invW = 1.0f / (float)g.W;
    for (int tile = t_first; tile < t_end; tile += t_step, ++it) {
      const int s = it % NSTAGE;
      const int m0 = tile * TC_BM;
      float4 cur[8];
      if (!A_PLANAR) {
#pragma unroll
        for (int r = 0; r < 8; ++r) cur[r] = pre[r];
        const int nt = tile + t_step;
        if (nt < t_end) {
          const float* a0 = g.A + gemm_src_row(g, nt * TC_BM) * TC_K;
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int row = rsub + 32 * (r & 3);
            const int chunk = chunk_lo + 8 * (r >> 2);
            pre[r] = (nt * TC_BM + row < g.M)
                         ? __ldg(reinterpret_cast<const float4*>(a0 + (size_t)row * TC_K + chunk * 4))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
      // warp-uniform exit: the lanes of a warp meet again at the __syncwarp before the arrive
      if (__any_sync(0xffffffffu, !tc::mbar_wait(&empty[s], ((it / NSTAGE) & 1) ^ 1))) { atomicExch(&g_tc_error, 1); break; }
      unsigned char* a_hi = smem + L::A_OFF + (uint32_t)s * 2u * TC_A_HALF;
      unsigned char* a_lo = a_hi + TC_A_HALF;
      if (!A_PLANAR) {
        int px0 = 0, t = 0;
        if (rot[0] || rot[1]) {
          const int fr = m0 / g.HW;
          px0 = m0 - fr * g.HW;
          t = gemm_rope_t(g, fr);
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int row = rsub + 32 * (r & 3);
          const int chunk = chunk_lo + 8 * (r >> 2);
          float4 v = cur[r];
          if (rot[r >> 2]) {
            const int px = px0 + row;
            const int h = (int)(((float)px + 0.5f) * invW);     // exact for px < 2^22
            const int w = px - h * g.W;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float2 ct = __ldg(&g.rope_t[t * 32 + chunk * 2 + e]);
              const float2 ch = __ldg(&g.rope_h[h * 32 + chunk * 2 + e]);
              const float2 cw = __ldg(&g.rope_w[w * 32 + chunk * 2 + e]);
              const float cx = ct.x * ch.x - ct.y * ch.y, sx = ct.x * ch.y + ct.y * ch.x;
              const float c2 = cx * cw.x - sx * cw.y, s2 = cx * cw.y + sx * cw.x;
              float& xe = e ? v.z : v.x;
              float& xo = e ? v.w : v.y;
              const float ne = xe * c2 - xo * s2, no = xe * s2 + xo * c2;
              xe = ne; xo = no;
            }
          }
          float4 h4, l4;
          tc::split_tf32(v.x, h4.x, l4.x); tc::split_tf32(v.y, h4.y, l4.y);
          tc::split_tf32(v.z, h4.z, l4.z); tc::split_tf32(v.w, h4.w, l4.w);
          const uint32_t off = (uint32_t)(chunk >> 3) * (TC_BM * 128u) + tc::sw128_offset(row, chunk & 7);
          *reinterpret_cast<float4*>(a_hi + off) = h4;
          *reinterpret_cast<float4*>(a_lo + off) = l4;
        }
      } else {
        // thread = (pixel row, K half); planes are contiguous over pixels, so each k is a
        // coalesced read across the lanes of a warp
        const int row = tid & 127, kh = tid >> 7, m = m0 + row;
        float v[32];
        if (m < g.M) {
          const int fo = m / g.HW, px = m - fo * g.HW;
          const int fr = gemm_src_frame(g, fo);
          const float* ap = g.A + ((size_t)fr * g.a_planes + g.a_plane0 + kh * 32) * g.HW + px;
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = __ldg(ap + (size_t)k * g.HW);
          if (g.rms_scale != nullptr) {
            // the other K half of the row is re-read (cache hit: the partner thread loads it)
            const float* op = g.A + ((size_t)fr * g.a_planes + g.a_plane0 + (1 - kh) * 32) * g.HW + px;
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) { const float o = op[(size_t)k * g.HW]; ss = fmaf(o, o, ss); }
#pragma unroll
            for (int k = 0; k < 32; ++k) ss = fmaf(v[k], v[k], ss);
            const float rinv = rsqrtf(ss * (1.0f / TC_K) + 1e-6f);
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] *= rinv * __ldg(&g.rms_scale[kh * 32 + k]);
          }
          if (g.gate != nullptr) {
            const float* gp = g.gate + ((size_t)(g.g_compact ? fo : fr) * g.g_planes + g.g_plane0 + kh * 32) * g.HW + px;
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] *= __ldg(gp + (size_t)k * g.HW);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = 0.f;
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float4 h4, l4;
          tc::split_tf32(v[4 * c + 0], h4.x, l4.x); tc::split_tf32(v[4 * c + 1], h4.y, l4.y);
          tc::split_tf32(v[4 * c + 2], h4.z, l4.z); tc::split_tf32(v[4 * c + 3], h4.w, l4.w);
          const uint32_t off = (uint32_t)kh * (TC_BM * 128u) + tc::sw128_offset(row, c);
          *reinterpret_cast<float4*>(a_hi + off) = h4;
          *reinterpret_cast<float4*>(a_lo + off) = l4;
        }
      }
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&full[s]);
    }
  } else if (warp == TC_MMA_WARP) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = tc::make_idesc_tf32(TC_BM, N);
      const uint32_t b_hi = sbase + L::B_OFF, b_lo = b_hi + L::B_HALF;
      int it = 0;
      bool ok = true;
      for (int tile = t_first; tile < t_end; tile += t_step, ++it) {
        const int s = it % NSTAGE, sph = (it / NSTAGE) & 1;    // A stage and its phase
        const int ac = it & 1, ph = (it >> 1) & 1;              // accumulator and its phase
        if (!tc::mbar_wait(&accempty[ac], ph ^ 1) || !tc::mbar_wait(&full[s], sph)) {
          atomicExch(&g_tc_error, 2); ok = false; break;
        }
        tc::fence_after_sync();
        const uint32_t a_hi = sbase + L::A_OFF + (uint32_t)s * 2u * TC_A_HALF, a_lo = a_hi + TC_A_HALF;
        const uint32_t d = tmem_base + (uint32_t)ac * N;
        uint32_t acc = 0;
#pragma unroll
        for (int pass = 0; pass < 3; ++pass) {
          const uint32_t ab = pass == 1 ? a_lo : a_hi;
          const uint32_t bb = pass == 2 ? b_lo : b_hi;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t koff = (uint32_t)(ks & 3) * 32u;
            const uint64_t ad = tc::make_desc_sw128(ab + (uint32_t)(ks >> 2) * (TC_BM * 128u) + koff);
            const uint64_t bd = tc::make_desc_sw128(bb + (uint32_t)(ks >> 2) * (N * 128u) + koff);
            tc::mma_tf32(d, ad, bd, idesc, acc);
            acc = 1;
          }
        }
        tc::commit(&empty[s]);
        tc::commit(&accfull[ac]);
      }
      // nothing of this thread's tensor work may be in flight when TMEM is freed
      tc::commit(done);
      if (!tc::mbar_wait(done, 0) && ok) atomicExch(&g_tc_error, 3);
    }
    __syncwarp();
  } else if (warp > TC_MMA_WARP) {
    // ================================ epilogue ================================
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - (TC_MMA_WARP + 1)) >> 2;   // which half of the N columns
    const int row = q * 32 + lane;
    int it = 0;
    for (int tile = t_first; tile < t_end; tile += t_step, ++it) {
      const int s = it & 1, ph = (it >> 1) & 1;
      bool ok = tc::mbar_wait(&accfull[s], ph);
      if (STG) {
        // the named barriers below need all 128 threads of the half: make the exit uniform
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, %2, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(all_ok) : "r"((uint32_t)ok), "r"(1 + half) : "memory");
        ok = all_ok != 0;
      } else {
        ok = !__any_sync(0xffffffffu, !ok);
      }
      if (!ok) { atomicExch(&g_tc_error, 4); break; }
      tc::fence_after_sync();
      const int m = tile * TC_BM + row;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)s * N;
#pragma unroll 1
      for (int cc = half * (N / 64); cc < (half + 1) * (N / 64); ++cc) {
        if (ZLAST && cc * 32 >= g.act_n0 && (m / g.HW) % g.T != g.T - 1) continue;   // tile-uniform
        uint32_t r[32];
        tc::ld_32x32b_x32(taddr + cc * 32, r);
        tc::wait_ld();
        if (STG) {
          // this half's 128 threads share two 16 KB staging chunks and named barrier 1 + half
          const int grp_tid = tid - (TC_MMA_WARP + 1 + 4 * half) * 32;      // 0..127
          float* stg = reinterpret_cast<float*>(smem + L::OUT_OFF) + half * 4096;
          // the TMA store that last read this chunk buffer must have drained it
          if (grp_tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
          const float* bs = bias_s + cc * 32;
          const int act = (g.out_act != 0 && cc * 32 >= g.act_n0) ? g.out_act : 0;
          if (!A_PLANAR) {
            // chunk layout [column j][pixel]: lanes write consecutive pixels (conflict-free)
            float vals[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float v = __uint_as_float(r[j]) + bs[j];
              if (act == 1) v = silu_f(v); else if (act == 2) v = sigmoid_f(v);
              vals[j] = v;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) stg[j * 128 + row] = vals[j];
          } else {
            // chunk layout [pixel][32 columns] in the 128-byte swizzle the tensor map expects
            float vals[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) vals[j] = __uint_as_float(r[j]) + bs[j];
            if (g.sub != nullptr) {
              const float4* sp = reinterpret_cast<const float4*>(g.sub + (size_t)m * g.N + cc * 32);
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 sv = __ldg(sp + (j >> 2));
                vals[j] -= sv.x; vals[j + 1] -= sv.y; vals[j + 2] -= sv.z; vals[j + 3] -= sv.w;
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(stg) +
                                         tc::sw128_offset(row, j >> 2)) =
                  make_float4(vals[j], vals[j + 1], vals[j + 2], vals[j + 3]);
          }
          tc::fence_proxy_async();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
          if (grp_tid == 0) {
            const int m0 = tile * TC_BM;
            if (!A_PLANAR) {
              const int fr = m0 / g.HW, px0 = m0 - fr * g.HW;
              tc::tma_store_3d(&omap, stg, px0, g.o_plane0 + cc * 32, fr);
            } else {
              tc::tma_store_2d(&omap, stg, cc * 32, m0);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          continue;
        }
        if (m < g.M) {
          if (!A_PLANAR) {
            // planar output: lanes = consecutive pixels -> 128-byte coalesced stores per column.
            // All 32 values are finished in registers before the first store: the stores go
            // through a generic pointer, so bias loads placed between them could not be hoisted.
            const int fr = m / g.HW, px = m - fr * g.HW;
            float* op = g.out + ((size_t)fr * g.o_planes + g.o_plane0 + cc * 32) * g.HW + px;
            const float* bs = bias_s + cc * 32;
            float vals[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) vals[j] = __uint_as_float(r[j]) + bs[j];
            if (g.out_act == 1 && cc * 32 >= g.act_n0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) vals[j] = silu_f(vals[j]);
            } else if (g.out_act == 2 && cc * 32 >= g.act_n0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) vals[j] = sigmoid_f(vals[j]);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) op[(size_t)j * g.HW] = vals[j];
          } else {
            float* op = g.out + (size_t)m * g.N + cc * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v;
              v.x = __uint_as_float(r[j + 0]) + bias_s[cc * 32 + j + 0];
              v.y = __uint_as_float(r[j + 1]) + bias_s[cc * 32 + j + 1];
              v.z = __uint_as_float(r[j + 2]) + bias_s[cc * 32 + j + 2];
              v.w = __uint_as_float(r[j + 3]) + bias_s[cc * 32 + j + 3];
              if (g.sub != nullptr) {
                const float4 sv = __ldg(reinterpret_cast<const float4*>(g.sub + (size_t)m * g.N + cc * 32 + j));
                v.x -= sv.x; v.y -= sv.y; v.z -= sv.z; v.w -= sv.w;
              }
              *reinterpret_cast<float4*>(op + j) = v;
            }
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&accempty[s]);
    }
    // shared memory must outlive the last TMA stores that read it
    if (STG) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == TC_MMA_WARP) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Whether the tensor-core kernel covers this problem (else the CUDA-core GEMM runs).
bool gemm_tc_supported(const GemmArgs& g, bool a_planar) {
  if (g.K != TC_K || (g.N != 64 && g.N != 128 && g.N != 192)) return false;
  if (g.HW % TC_BM != 0 || g.M % TC_BM != 0) return false;
  if (g.out_act != 0 && g.act_n0 % 32 != 0) return false;
  if (a_planar && g.N == 192) return false;
  return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of the GEMM output for the TMA-store epilogue: 16 KB boxes of 128 pixels x 32 columns.
static bool make_out_map(const GemmArgs& g, bool a_planar, CUtensorMap* map) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint32_t es[3] = {1, 1, 1};
  CUresult r;
  if (!a_planar) {
    const cuuint64_t dims[3] = {(cuuint64_t)g.HW, (cuuint64_t)g.o_planes, (cuuint64_t)(g.M / g.HW)};
    const cuuint64_t strides[2] = {(cuuint64_t)g.HW * 4, (cuuint64_t)g.o_planes * g.HW * 4};
    const cuuint32_t box[3] = {128, 32, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, g.out, dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    const cuuint64_t dims[2] = {(cuuint64_t)g.N, (cuuint64_t)g.M};
    const cuuint64_t strides[1] = {(cuuint64_t)g.N * 4};
    const cuuint32_t box[2] = {32, 128};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, g.out, dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS;
}

template <int N, bool A_PLANAR, bool STG, bool ZLAST = false>
static int launch_tc_v(const GemmArgs& g, const CUtensorMap& map, cudaStream_t st) {
  const int num_tiles = g.M / TC_BM;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const int grid = num_tiles < sms ? num_tiles : sms;
  const size_t smem = TcSmem<N, STG>::TOTAL + 1024;      // slack for the 1024-byte alignment
  e = cudaFuncSetAttribute(gemm_tc_kernel<N, A_PLANAR, STG, ZLAST>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  gemm_tc_kernel<N, A_PLANAR, STG, ZLAST><<<grid, TC_THREADS, smem, st>>>(g, num_tiles, map);
  return check_launch();
}

template <int N, bool A_PLANAR>
static int launch_tc(const GemmArgs& g, cudaStream_t st) {
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  // TMA-store epilogue for the channels-last output (planar A) unless the driver entry point is
  // missing.  For the planar output it measured slower than direct stores (2.1 ms vs 1.44 ms on
  // the in_proj of cfg2), so that direction keeps direct stores.
  const bool stg = A_PLANAR && N <= 128 && (reinterpret_cast<uintptr_t>(g.out) & 15u) == 0 &&
                   make_out_map(g, A_PLANAR, &map);
  if (N <= 128 && stg) return launch_tc_v<N, A_PLANAR, (N <= 128)>(g, map, st);
  return launch_tc_v<N, A_PLANAR, false>(g, map, st);
}

int launch_gemm_tc(const GemmArgs& g, bool a_planar, cudaStream_t st) {
  if (!gemm_tc_supported(g, a_planar)) return CSSM_ERR_UNSUPPORTED;
  if (g.z_last_only && !a_planar && g.N == 128) {
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    return launch_tc_v<128, false, false, true>(g, map, st);
  }
  if (!a_planar)
    return g.N == 192 ? launch_tc<192, false>(g, st)
                      : g.N == 128 ? launch_tc<128, false>(g, st) : launch_tc<64, false>(g, st);
  return g.N == 128 ? launch_tc<128, true>(g, st) : launch_tc<64, true>(g, st);
}

int read_tc_error(int* out, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_tc_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  }
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

}  // namespace cssm

extern "C" {
int cssm_device_error(int* out, int clear) {
  if (!out) return CSSM_ERR_NULL;
  int a = 0, b = 0;
  int rc = cssm::read_tc_error(&a, clear);
  if (rc != CSSM_OK) return rc;
  rc = cssm::read_spec_error(&b, clear);
  if (rc != CSSM_OK) return rc;
  int c = 0, m = 0;
  rc = cssm::read_bf16_error(&c, clear);
  if (rc != CSSM_OK) return rc;
  rc = cssm::read_mlp_error(&m, clear);
  // low byte: fp32 tensor-core GEMMs, next byte: fused spectral kernels, third: bf16 GEMM, fourth: fused MLP
  *out = a | (b << 8) | (c << 16) | (m << 24);
  return rc;
}
}
