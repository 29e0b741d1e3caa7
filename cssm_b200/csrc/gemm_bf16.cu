// bf16 tcgen05 / TMEM GEMM with a K loop, for the channel contractions of the CSSM-SHViT model
// (Dense layers with K = 64 ... 1536, and the 3x3 stride-2 ConvBN layers as implicit GEMMs).
//
//   out[m, n] = act( sum_k A[m, k] * Wt[n, k] + bias[n] ) (+ res[m, n]),  bf16 in, fp32 accumulate.
//
// Persistent kernel, one CTA per SM, 320 threads (448 in conv mode), warp-specialised:
//   warp 0     TMA producer: one lane issues cp.async.bulk.tensor loads of the A tile (128 rows x
//              64 k, plain mode) and the weight tile (BN rows x 64 k) of every K block into a
//              4-stage ring of 128-byte-swizzled K-major operand tiles;
//   warp 1     MMA issuer: one lane issues 4 tcgen05.mma.kind::f16 (M128 x BN x K16) per K block
//              into one of four TMEM accumulators (BN <= 128; two for wider single tiles);
//              tcgen05.commit frees the stage / publishes the accumulator;
//   warps 2-9  epilogue, two warps per TMEM lane quadrant: tcgen05.ld (lane = output row), bias,
//              GELU / SiLU, residual; each half (one warp per quadrant) owns every other tile and two
//              of the accumulators, stages boxes of 128 rows x 64 bf16 columns in the 128-byte
//              swizzle in a ring of three or four slots and writes them with TMA tensor stores; the
//              residual box is fetched by TMA into the slot it will be staged in, two boxes ahead,
//              and added in place (N a multiple of 64; otherwise direct 16-byte loads and stores);
//   warps 10-13 im2col producers (conv mode only): eight consecutive lanes fetch the eight 16-byte
//              channel chunks of one output pixel's K block from the channels-last input (zero
//              outside the image), four pixels per warp instruction, and write them in the same
//              swizzled layout; the loads of the next two K blocks are in flight meanwhile.
// Every mbarrier wait is bounded; on expiry the kernel records an error code (cssm_device_error)
// and winds down.  No multicast, no cluster: each CTA loads its own tiles.
#include <cuda.h>
#include <cuda_bf16.h>
#include <string.h>
#include "kernels.cuh"
#include "tc05.cuh"
#include "bf16_ops.cuh"

namespace cssm {

__device__ int g_bf16_error = 0;

constexpr int GB_THREADS_PLAIN = 320, GB_THREADS_CONV = 448;
constexpr int GB_BM = 128, GB_BK = 64, GB_MAX_STAGES = 4;
constexpr uint32_t GB_A_BYTES = GB_BM * 128u;            // one A stage: 128 rows x 128 bytes

__device__ __forceinline__ uint32_t make_idesc_bf16(uint32_t M, uint32_t N) {
  uint32_t d = 0;
  d |= 1u << 4;            // D format: f32
  d |= 1u << 7;            // A format: bf16
  d |= 1u << 10;           // B format: bf16
  d |= (N >> 3) << 17;     // N / 8
  d |= (M >> 4) << 24;     // M / 16
  return d;
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// RTMA (with TMA_OUT): the residual boxes come by TMA into the staging slots.
template <bool IM2COL, bool TMA_OUT, bool RTMA>
__global__ void __launch_bounds__(IM2COL ? GB_THREADS_CONV : GB_THREADS_PLAIN, 1)
gemm_bf16_kernel(const Bf16GemmArgs g, const __grid_constant__ CUtensorMap amap,
                 const __grid_constant__ CUtensorMap bmap, const __grid_constant__ CUtensorMap omap,
                 const __grid_constant__ CUtensorMap rmap) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = tc::smem_u32(smem);
  const uint32_t BN = (uint32_t)g.BN;
  // wres: the whole weight matrix (one N tile, all K blocks) stays in shared memory for the life of
  // the CTA and the ring carries only the A tiles
  const bool wres = g.wres != 0;
  const uint32_t wres_bytes = wres ? (uint32_t)(g.Kpad / GB_BK) * BN * 128u : 0u;
  const uint32_t stage_bytes = GB_A_BYTES + (wres ? 0u : BN * 128u);
  const int NS = g.stages;                                  // ring depth (3 when BN = 256 and TMA_OUT)
  unsigned char* ring = smem + wres_bytes;
  unsigned char* out_s = ring + (uint32_t)NS * stage_bytes; // TMA_OUT: 2 x ostg staging boxes of 16 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_s + (TMA_OUT ? (uint32_t)(2 * g.ostg) * 16384u : 0u));
  uint64_t* full = bars;                        // [4] operands landed
  uint64_t* empty = bars + GB_MAX_STAGES;       // [4] stage consumed
  uint64_t* accfull = bars + 2 * GB_MAX_STAGES; // [4] accumulator complete
  uint64_t* accempty = accfull + 4;             // [4] accumulator drained
  uint64_t* resfull = accempty + 4;             // [2][4] residual box landed in its staging slot
  uint64_t* done = resfull + 8;
  uint64_t* wfull = done + 1;                   // resident weights landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wfull + 1);
  const int NACC = g.nacc;                                  // TMEM accumulators: 4 of BN <= 128 columns, else 2

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = g.N / g.BN;
  const int m_tiles = g.conv_tma ? g.tiles_w * g.tiles_h * ((g.Bimg + g.Bbox - 1) / g.Bbox) : (g.M + GB_BM - 1) / GB_BM;
  const int num_tiles = m_tiles * n_tiles;
  const int kblocks = g.Kpad / GB_BK;
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)NACC * BN) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      tc::mbar_init(&full[s], IM2COL ? 1 + 4 : 1);      // TMA lane + one lane per producer warp
      tc::mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 4; ++a) {
      tc::mbar_init(&accfull[a], 1);
      // one lane per warp of the half that drains the accumulator
      tc::mbar_init(&accempty[a], 4);
    }
    for (int a = 0; a < 8; ++a) tc::mbar_init(&resfull[a], 1);
    tc::mbar_init(done, 1);
    tc::mbar_init(wfull, 1);
    tc::fence_mbar_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool bad = false;

  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      if (wres) {
        tc::mbar_expect_tx(wfull, wres_bytes);
        for (int kb = 0; kb < kblocks; ++kb) tc::tma_load_2d(smem + (uint32_t)kb * BN * 128u, &bmap, kb * GB_BK, 0, wfull);
      }
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !bad; tile += gridDim.x) {
        const int mt = tile / n_tiles;
        const int m0 = mt * GB_BM, n0 = (tile % n_tiles) * g.BN;
        // conv through TMA: the tile's patch origin (input coordinates of window position (0,0))
        int cw0 = 0, ch0 = 0, cb0 = 0;
        if (g.conv_tma) {
          const int tw = mt % g.tiles_w, th = (mt / g.tiles_w) % g.tiles_h;
          cb0 = (mt / (g.tiles_w * g.tiles_h)) * g.Bbox;
          cw0 = tw * g.Wbox * (g.conv_tma == 2 ? 1 : g.stride) - (g.conv_tma == 2 ? 0 : g.pad_w);
          ch0 = th * g.Hbox * g.stride - g.pad_h;
        }
        const uint32_t a_bytes = g.conv_tma ? (uint32_t)(g.Wbox * g.Hbox * g.Bbox) * 128u : GB_A_BYTES;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NS;
          if (!tc::mbar_wait(&empty[s], ((it / NS) & 1) ^ 1)) { atomicExch(&g_bf16_error, 5); bad = true; break; }
          unsigned char* a_s = ring + (uint32_t)s * stage_bytes;
          unsigned char* b_s = a_s + GB_A_BYTES;
          tc::mbar_expect_tx(&full[s], (IM2COL ? 0u : a_bytes) + (wres ? 0u : BN * 128u));
          if (g.conv_tma) {
            const int pos = kb / g.kb_per_tap, cb = kb - pos * g.kb_per_tap;
            const int pr = pos / g.pos_w, pc = pos - pr * g.pos_w;
            tc::tma_load_4d(a_s, &amap, cb * GB_BK, cw0 + pc, ch0 + pr, cb0, &full[s]);
          } else if (!IM2COL) {
            tc::tma_load_2d(a_s, &amap, kb * GB_BK, m0, &full[s]);
          }
          if (!wres) tc::tma_load_2d(b_s, &bmap, kb * GB_BK, n0, &full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(GB_BM, BN);
      if (wres && !tc::mbar_wait(wfull, 0)) { atomicExch(&g_bf16_error, 6); bad = true; }
      int it = 0, tcnt = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !bad; tile += gridDim.x, ++tcnt) {
        const int ac = tcnt % NACC, aph = (tcnt / NACC) & 1;
        if (!tc::mbar_wait(&accempty[ac], aph ^ 1)) { atomicExch(&g_bf16_error, 6); bad = true; break; }
        tc::fence_after_sync();
        const uint32_t d = tmem_base + (uint32_t)ac * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % NS;
          if (!tc::mbar_wait(&full[s], (it / NS) & 1)) { atomicExch(&g_bf16_error, 6); bad = true; break; }
          tc::fence_after_sync();
          const uint32_t a_s = sbase + wres_bytes + (uint32_t)s * stage_bytes;
          const uint32_t b_s = wres ? sbase + (uint32_t)kb * BN * 128u : a_s + GB_A_BYTES;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = tc::make_desc_sw128(a_s + (uint32_t)ks * 32u);
            const uint64_t bd = tc::make_desc_sw128(b_s + (uint32_t)ks * 32u);
            mma_bf16(d, ad, bd, idesc, (kb | ks) ? 1u : 0u);
          }
          tc::commit(&empty[s]);
        }
        if (bad) break;
        tc::commit(&accfull[ac]);
      }
      // nothing of this thread's tensor work may be in flight when TMEM is freed
      tc::commit(done);
      if (!tc::mbar_wait(done, 0) && !bad) atomicExch(&g_bf16_error, 7);
    }
    __syncwarp();
  } else if (warp < 10) {
    // ================================ epilogue ================================
    // Two halves of four warps (one per TMEM lane quadrant).  Half h owns the tiles of its CTA with
    // tile count parity h; accumulator = tile count mod NACC, so a half drains one accumulator while
    // the MMA warp fills its other one.
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    // bias, activation on 32 accumulator columns starting at tile column c0
    auto act32 = [&](const uint32_t (&r)[32], int n, float (&v)[32]) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      if (g.bias != nullptr) {
        const float4* bp = reinterpret_cast<const float4*>(g.bias + n);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 b4 = __ldg(bp + (j >> 2));
          v[j] += b4.x; v[j + 1] += b4.y; v[j + 2] += b4.z; v[j + 3] += b4.w;
        }
      }
      if (g.act == 1) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) gelu_tanh_x2(v[j], v[j + 1]);
      } else if (g.act == 2) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) silu_tanh_x2(v[j], v[j + 1]);
      }
    };
    if constexpr (TMA_OUT) {
      // Output boxes of 128 rows x 64 bf16 columns are staged in the 128-byte swizzle in a ring of D
      // slots per half and written by TMA tensor stores.  A residual is fetched by TMA into the
      // very slot its box will be staged in, D - 2 boxes ahead (the wait before a slot is reused
      // leaves only the most recent store pending), and is added in place.
      // (Both halves draining every tile of a two-accumulator configuration, each every other box,
      // measured slower than whole tiles in turn: 232 against 197 us for M = 1.6 M, K = 64, N = 256.)
      const bool issuer = q == 0 && lane == 0;    // issues this half's TMA loads and stores
      const int D = g.ostg, nb = g.BN / 64;
      constexpr int b0 = 0, bstep = 1, tstep = 2;
      const int t0 = half;
      unsigned char* stgh = out_s + (uint32_t)(half * D) * 16384u;
      uint64_t* resf = resfull + half * 4;
      constexpr bool rtma = RTMA;
      const bool rreg = !RTMA && g.res != nullptr;      // residual rows by plain loads
      int pf_t = t0, pf_box = b0, pf_q = 0;       // issuer: the next box whose residual is to be fetched
      auto pf_issue = [&]() {
        const int tile = blockIdx.x + pf_t * (int)gridDim.x;
        if (tile >= num_tiles) return;
        const int slot = pf_q % D;
        tc::mbar_expect_tx(&resf[slot], 16384u);
        tc::tma_load_2d(stgh + (uint32_t)slot * 16384u, &rmap, (tile % n_tiles) * g.BN + pf_box * 64,
                        (tile / n_tiles) * GB_BM, &resf[slot]);
        ++pf_q;
        pf_box += bstep;
        if (pf_box >= nb) { pf_box = b0; pf_t += tstep; }
      };
      if (rtma && issuer)
        for (int k = 0; k < D - 2; ++k) pf_issue();
      // all 128 threads of the half agree on `ok` (and meet, as a barrier)
      auto all_ok = [&](bool ok) {
        uint32_t r;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, %2, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(r) : "r"((uint32_t)ok), "r"(1 + half) : "memory");
        return r != 0;
      };
      int bq = 0;                                 // boxes staged by this half so far
      bool live = true;
      for (int tcnt = t0; live; tcnt += tstep) {
        const int tile = blockIdx.x + tcnt * (int)gridDim.x;
        if (tile >= num_tiles) break;
        const int m0 = (tile / n_tiles) * GB_BM, n0 = (tile % n_tiles) * g.BN;
        const int ac = tcnt % NACC, aph = (tcnt / NACC) & 1;
        const bool has_res = rreg && m0 + row < g.M;
        const uint4* rrow = reinterpret_cast<const uint4*>(g.res + (has_res ? (size_t)(m0 + row) * g.ldr + n0 : 0));
        uint4 rs[8];                              // rreg: residual of the next 64 columns
        auto fetch_res = [&](int c0) {
#pragma unroll
          for (int j = 0; j < 8; ++j) rs[j] = has_res ? __ldg(rrow + (c0 >> 3) + j) : make_uint4(0u, 0u, 0u, 0u);
        };
        if (rreg) fetch_res(0);
        if (!all_ok(tc::mbar_wait(&accfull[ac], aph))) { atomicExch(&g_bf16_error, 8); break; }
        tc::fence_after_sync();
        const uint32_t taddr = tlane + (uint32_t)ac * BN;
        uint32_t ra[32];
        for (int box = b0; box < nb; box += bstep, ++bq) {
          const int slot = bq % D;
          unsigned char* stg = stgh + (uint32_t)slot * 16384u;
          // residual by TMA: its box landed in this slot two boxes ago (a wait that expires is
          // recorded and the data is wrong, but every thread still meets the barriers below)
          if (rtma && !tc::mbar_wait(&resf[slot], (bq / D) & 1)) atomicExch(&g_bf16_error, 8);
          // accumulator -> bias, activation, residual -> eight packed 16-byte chunks.  Nothing here
          // writes the slot, so it runs while the earlier stores drain.  (Keeping the TMEM load of the
          // next 32 columns in flight during the arithmetic measured slower.)
          uint4 pk[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            float v[32];
            tc::ld_32x32b_x32(taddr + box * 64 + hh * 32, ra);
            tc::wait_ld();
            act32(ra, n0 + box * 64 + hh * 32, v);
            if (rtma || rreg) {
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                float f[8];
                unpack8(rtma ? *reinterpret_cast<const uint4*>(stg + tc::sw128_offset(row, hh * 4 + j4))
                             : rs[hh * 4 + j4], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j4 * 8 + e] += f[e];
              }
            }
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float f[8] = {v[j4 * 8], v[j4 * 8 + 1], v[j4 * 8 + 2], v[j4 * 8 + 3],
                                  v[j4 * 8 + 4], v[j4 * 8 + 5], v[j4 * 8 + 6], v[j4 * 8 + 7]};
              pk[hh * 4 + j4] = pack8(f);
            }
          }
          if (issuer) {
            // the store that last read the slot about to be refilled has drained: with a residual
            // that slot is the one of two boxes back, else this box's own (D boxes back)
            if (rtma || D < 3) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else if (D == 3) asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
            if (rtma) pf_issue();
          }
          // without the TMA residual the slot's last reader is only known to the issuer; with it
          // every thread rewrites just its own row of the box it has read
          if (!rtma) asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
          if (rreg && box + 1 < nb) fetch_res((box + 1) * 64);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(stg + tc::sw128_offset(row, c)) = pk[c];
          tc::fence_proxy_async();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
          if (issuer) {
            if (g.conv_tma) {
              const int mt = tile / n_tiles;
              const int tw = mt % g.tiles_w, th = (mt / g.tiles_w) % g.tiles_h;
              tc::tma_store_4d(&omap, stg, n0 + box * 64, tw * g.Wbox, th * g.Hbox,
                               (mt / (g.tiles_w * g.tiles_h)) * g.Bbox);
            } else {
              tc::tma_store_2d(&omap, stg, n0 + box * 64, m0);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (!live) break;
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&accempty[ac]);
      }
      // the staging slots must outlive the last TMA stores that read them
      if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
      // direct 16-byte stores (N not a multiple of 64, or no tensor map): residual rows by plain loads
      for (int i = 0;; ++i) {
        const int tcnt = 2 * i + half;
        const int tile = blockIdx.x + tcnt * (int)gridDim.x;
        if (tile >= num_tiles) break;
        const int m0 = (tile / n_tiles) * GB_BM, n0 = (tile % n_tiles) * g.BN;
        const int ac = tcnt % NACC, aph = (tcnt / NACC) & 1;
        const int m = m0 + row;
        const bool has_res = g.res != nullptr && m < g.M;
        const uint4* rrow = reinterpret_cast<const uint4*>(g.res + (has_res ? (size_t)m * g.ldr + n0 : 0));
        uint4 rs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) rs[j] = has_res ? __ldg(rrow + j) : make_uint4(0u, 0u, 0u, 0u);
        if (__any_sync(0xffffffffu, !tc::mbar_wait(&accfull[ac], aph))) { atomicExch(&g_bf16_error, 8); break; }
        tc::fence_after_sync();
        const uint32_t taddr = tlane + (uint32_t)ac * BN;
        uint32_t ra[32];
        for (int c0 = 0; c0 < g.BN; c0 += 32) {
          float v[32];
          tc::ld_32x32b_x32(taddr + c0, ra);
          tc::wait_ld();
          act32(ra, n0 + c0, v);
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            float f[8];
            unpack8(rs[j4], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j4 * 8 + e] += f[e];
          }
          if (c0 + 32 < g.BN) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              rs[j] = has_res ? __ldg(rrow + ((c0 + 32) >> 3) + j) : make_uint4(0u, 0u, 0u, 0u);
          }
          if (m < g.M) {
            uint4* op = reinterpret_cast<uint4*>(g.out + (size_t)m * g.ldo + n0 + c0);
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float f[8] = {v[j4 * 8], v[j4 * 8 + 1], v[j4 * 8 + 2], v[j4 * 8 + 3],
                                  v[j4 * 8 + 4], v[j4 * 8 + 5], v[j4 * 8 + 6], v[j4 * 8 + 7]};
              op[j4] = pack8(f);
            }
          }
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&accempty[ac]);
      }
    }
  } else if (IM2COL) {
    // ================================ im2col producers ================================
    // lane = (row group rg, chunk c): the eight lanes of a group read the eight 16-byte chunks of one
    // output pixel's K block (contiguous channels of one or two taps); thread handles rows rg + 16 i.
    const int pt = tid - 10 * 32;                 // 0..127
    const int c = pt & 7, rg = pt >> 3;
    const int HWo = g.Ho * g.Wo;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !bad; tile += gridDim.x) {
      const int mt = (tile / n_tiles) * GB_BM;
      int hi0[8], wi0[8], pb[8];                    // window origin and first pixel of the image
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = mt + rg + 16 * i;
        const bool live = m < g.M;
        const int b = live ? m / HWo : 0;
        const int px = live ? m - b * HWo : 0;
        const int ho = px / g.Wo, wo = px - ho * g.Wo;
        hi0[i] = live ? ho * g.stride - g.pad_h : -100000;     // dead rows fail the bounds test
        wi0[i] = wo * g.stride - g.pad_w;
        pb[i] = b * g.Hi * g.Wi;
      }
      auto gather = [&](int kb, uint4 (&v)[8]) {
        const int k0 = kb * GB_BK + c * 8;
        const int tap = k0 / g.Cin, c0 = k0 - tap * g.Cin;
        const int ti = tap / g.ksz, tj = tap - ti * g.ksz;
        const bool kin = kb < kblocks && k0 < g.K;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int hi = hi0[i] + ti, wi = wi0[i] + tj;
          const bool in = kin && hi >= 0 && hi < g.Hi && wi >= 0 && wi < g.Wi;
          v[i] = in ? __ldg(reinterpret_cast<const uint4*>(g.A + (size_t)(pb[i] + hi * g.Wi + wi) * g.Cin + c0))
                    : make_uint4(0u, 0u, 0u, 0u);
        }
      };
      // register ring two K blocks deep
      uint4 r0[8], r1[8], r2[8];
      gather(0, r0);
      gather(1, r1);
      for (int kb = 0; kb < kblocks && !bad; kb += 3) {
        // three blocks per trip so that the ring slots keep compile-time names
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          if (kb + u >= kblocks) break;
          uint4 (&cur)[8] = u == 0 ? r0 : (u == 1 ? r1 : r2);
          uint4 (&nxt)[8] = u == 0 ? r2 : (u == 1 ? r0 : r1);
          gather(kb + u + 2, nxt);
          const int s = it % NS;
          if (__any_sync(0xffffffffu, !tc::mbar_wait(&empty[s], ((it / NS) & 1) ^ 1))) { atomicExch(&g_bf16_error, 9); bad = true; break; }
          unsigned char* a_s = ring + (uint32_t)s * stage_bytes;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(a_s + tc::sw128_offset(rg + 16 * i, c)) = cur[i];
          tc::fence_proxy_async();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&full[s]);
          ++it;
        }
      }
    }
  }
  // error path only: give copies that may still be in flight a bounded time to land
  if (bad)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, tmem_cols);
  }
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

// K-major bf16 matrix [rows][kcols] (row stride ld elements) -> boxes of 64 k x box_rows rows
static bool make_kmajor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t kcols,
                            uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {kcols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {64, box_rows}, es[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int read_bf16_error(int* out, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_bf16_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_bf16_error, &zero, sizeof(int));
  }
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

// Tile width: 256, 192, 128 or 64 columns with the TMA-store epilogue;
// other multiples of 32 up to 256 as one tile with direct stores.
int gemm_bf16_pick_bn(int N) {
  if (N % 256 == 0) return 256;
  if (N % 192 == 0) return 192;
  if (N % 128 == 0) return 128;
  if (N % 64 == 0) return 64;
  if (N <= 256 && N % 32 == 0) return N;
  return 0;
}

// (rows x cols) bf16 output with row stride ld -> boxes of 64 columns x 128 rows for the TMA stores
static bool make_out_map(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {64, 128}, es[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-D bf16 tensor (d0 innermost) with byte strides st[0..2] of dims 1..3, boxes and traversal strides
static bool make_map_4d(CUtensorMap* map, const void* base, const uint64_t (&dims)[4], const uint64_t (&st)[3],
                        const uint32_t (&box)[4], const uint32_t (&es)[4]) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  const cuuint64_t s[3] = {st[0], st[1], st[2]};
  const cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  const cuuint32_t e[4] = {es[0], es[1], es[2], es[3]};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), d, s, b, e,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int conv3x3s2_weight_layout(int Cin, int Wi, int Cout) { return (Cin == 32 && Wi % 2 == 0 && Cout % 64 == 0) ? 1 : 0; }
int conv3x3s2_packed_k(int Cin, int Wi, int Cout) { return conv3x3s2_weight_layout(Cin, Wi, Cout) ? 384 : 9 * Cin; }

int launch_gemm_bf16(Bf16GemmArgs g, cudaStream_t st) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return CSSM_ERR_DIMS;
  const bool conv = g.ksz > 0;
  const int wide = conv ? conv3x3s2_weight_layout(g.Cin, g.Wi, g.N) : 0;
  // 3x3 stride-2 convs with 64-channel K blocks go through strided TMA boxes (no gather warps)
  g.conv_tma = 0;
  if (conv && g.ksz == 3 && g.stride == 2 && g.N % 64 == 0 && g.res == nullptr && (wide || g.Cin % 64 == 0))
    g.conv_tma = wide ? 2 : 1;
  const int Kw = conv ? conv3x3s2_packed_k(g.Cin, g.Wi, g.N) : g.K;      // K as the packed weights lay it out
  g.Kpad = (Kw + GB_BK - 1) / GB_BK * GB_BK;
  g.BN = gemm_bf16_pick_bn(g.N);
  // a residual with a short K loop gains more from the TMA residual prefetch (three staging slots,
  // BN <= 128) than it loses in operand traffic: 37 against 47 us for M = 100 K, K = 256, N = 256
  if (g.BN == 256 && g.res != nullptr && g.K < 512) g.BN = 128;
  if (g.BN == 0 || g.ldw < g.Kpad || (g.ldw % 8) != 0) return CSSM_ERR_UNSUPPORTED;
  if (g.ldo % 8 != 0 || (g.res != nullptr && g.ldr % 8 != 0)) return CSSM_ERR_UNSUPPORTED;
  if (!aligned16(g.A) || !aligned16(g.Wt) || (g.out && !aligned16(g.out)) ||
      (g.out_f32 && !aligned16(g.out_f32)) || (g.res && !aligned16(g.res)))
    return CSSM_ERR_ALIGN;
  if (g.out_f32 != nullptr || g.out == nullptr) return CSSM_ERR_UNSUPPORTED;
  const bool im2col = conv && !g.conv_tma;
  if (conv) {
    if (g.Cin % 8 != 0 || g.K != g.ksz * g.ksz * g.Cin) return CSSM_ERR_UNSUPPORTED;
    if (wide && !g.conv_tma) return CSSM_ERR_UNSUPPORTED;          // the wide weight layout has no gather path
  } else if (g.K % 8 != 0 || g.lda % 8 != 0 || g.lda < g.K) {
    return CSSM_ERR_UNSUPPORTED;
  }
  CUtensorMap amap, bmap, omap, rmap;
  memset(&amap, 0, sizeof(amap));
  memset(&bmap, 0, sizeof(bmap));
  memset(&omap, 0, sizeof(omap));
  memset(&rmap, 0, sizeof(rmap));
  bool tma_out = g.BN % 64 == 0;
  int m_tiles = (g.M + GB_BM - 1) / GB_BM;
  if (g.conv_tma) {
    // M tile = Bbox images x Hbox output rows x Wbox output columns, at most 128 pixels
    g.Bimg = g.M / (g.Ho * g.Wo);
    g.tiles_w = (g.Wo + 127) / 128;
    g.Wbox = (g.Wo + g.tiles_w - 1) / g.tiles_w;
    const int hmax = 128 / g.Wbox > 0 ? 128 / g.Wbox : 1;
    g.tiles_h = (g.Ho + hmax - 1) / hmax;
    g.Hbox = (g.Ho + g.tiles_h - 1) / g.tiles_h;
    g.Bbox = (g.tiles_w == 1 && g.tiles_h == 1) ? 128 / (g.Wbox * g.Hbox) : 1;
    if (g.Bbox > g.Bimg) g.Bbox = g.Bimg;
    if (g.Bbox < 1) g.Bbox = 1;
    m_tiles = g.tiles_w * g.tiles_h * ((g.Bimg + g.Bbox - 1) / g.Bbox);
    const uint64_t C = (uint64_t)g.Cin;
    bool ok;
    if (g.conv_tma == 2) {
      // pairs of adjacent input pixels as 64-channel "wide pixels": window columns {0,1} and {2,(3)}
      const uint64_t W2 = (uint64_t)g.Wi / 2;
      const uint64_t dims[4] = {64, W2, (uint64_t)g.Hi, (uint64_t)g.Bimg};
      const uint64_t stb[3] = {128, W2 * 128, (uint64_t)g.Hi * W2 * 128};
      const uint32_t box[4] = {64, (uint32_t)g.Wbox, (uint32_t)g.Hbox * 2, (uint32_t)g.Bbox};
      const uint32_t es[4] = {1, 1, 2, 1};
      ok = make_map_4d(&amap, g.A, dims, stb, box, es);
      g.kb_per_tap = 1; g.pos_w = 2;
    } else {
      const uint64_t dims[4] = {C, (uint64_t)g.Wi, (uint64_t)g.Hi, (uint64_t)g.Bimg};
      const uint64_t stb[3] = {C * 2, (uint64_t)g.Wi * C * 2, (uint64_t)g.Hi * g.Wi * C * 2};
      const uint32_t box[4] = {64, (uint32_t)g.Wbox * 2, (uint32_t)g.Hbox * 2, (uint32_t)g.Bbox};
      const uint32_t es[4] = {1, 2, 2, 1};
      ok = make_map_4d(&amap, g.A, dims, stb, box, es);
      g.kb_per_tap = g.Cin / 64; g.pos_w = 3;
    }
    const uint64_t N = (uint64_t)g.N;
    const uint64_t odims[4] = {N, (uint64_t)g.Wo, (uint64_t)g.Ho, (uint64_t)g.Bimg};
    const uint64_t ost[3] = {(uint64_t)g.ldo * 2, (uint64_t)g.Wo * g.ldo * 2, (uint64_t)g.Ho * g.Wo * g.ldo * 2};
    const uint32_t obox[4] = {64, (uint32_t)g.Wbox, (uint32_t)g.Hbox, (uint32_t)g.Bbox};
    const uint32_t oes[4] = {1, 1, 1, 1};
    ok = ok && make_map_4d(&omap, g.out, odims, ost, obox, oes);
    if (!ok) return CSSM_ERR_CUDA;
  } else {
    // A: out-of-range k columns (K < Kpad) and rows (M not a multiple of 128) arrive as zeros
    if (!im2col && !make_kmajor_map(&amap, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, GB_BM))
      return CSSM_ERR_CUDA;
    tma_out = tma_out && make_out_map(&omap, g.out, (uint64_t)g.M, (uint64_t)g.N, (uint64_t)g.ldo);
    if (tma_out && g.res != nullptr && g.BN <= 128)
      tma_out = make_out_map(&rmap, const_cast<__nv_bfloat16*>(g.res), (uint64_t)g.M, (uint64_t)g.N, (uint64_t)g.ldr);
  }
  if (!make_kmajor_map(&bmap, g.Wt, (uint64_t)g.N, (uint64_t)g.Kpad, (uint64_t)g.ldw, (uint32_t)g.BN))
    return CSSM_ERR_CUDA;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const int tiles = m_tiles * (g.N / g.BN);
  const int grid = tiles < sms ? tiles : sms;
  // Weights of at most 64 KB that form a single N tile stay resident in shared memory (a weight tile
  // re-read from L2 for every M tile costs as much operand traffic as the A tile itself).
  const size_t wres_bytes = (size_t)g.Kpad * g.BN * 2;
  g.wres = (!im2col && g.N == g.BN && wres_bytes <= 64 * 1024) ? 1 : 0;
  const size_t stage = GB_A_BYTES + (g.wres ? 0 : (size_t)g.BN * 128u);
  const size_t budget = 227 * 1024 - (g.wres ? wres_bytes : 0), fixed = 256 + 1024;
  // Residual by TMA (plain GEMMs with tiles of at most 128 columns): four accumulators and three or
  // four staging slots per epilogue half.  Everything else: two accumulators, two slots, residual
  // rows (if any) by plain loads -- the configuration that measured best without a residual.
  const bool rtma = tma_out && g.res != nullptr && !conv && g.BN <= 128;
  g.nacc = rtma ? 4 : 2;
  g.stages = GB_MAX_STAGES;
  g.ostg = 0;
  if (tma_out) {
    while (g.stages > 2 && g.stages * stage + 4 * 16384 + fixed > budget) --g.stages;
    g.ostg = rtma ? (int)((budget - fixed - g.stages * stage) / (2 * 16384)) : 2;
    if (g.ostg > 4) g.ostg = 4;
    if (g.ostg < (rtma ? 3 : 2)) return CSSM_ERR_UNSUPPORTED;
  } else {
    while (g.stages > 2 && g.stages * stage + fixed > budget) --g.stages;
  }
  const size_t smem = (g.wres ? wres_bytes : 0) + g.stages * stage + (size_t)g.ostg * 2 * 16384 + fixed;
  auto kern = im2col ? (tma_out ? gemm_bf16_kernel<true, true, false> : gemm_bf16_kernel<true, false, false>)
                     : (tma_out ? (rtma ? gemm_bf16_kernel<false, true, true> : gemm_bf16_kernel<false, true, false>)
                                : gemm_bf16_kernel<false, false, false>);
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  kern<<<grid, im2col ? GB_THREADS_CONV : GB_THREADS_PLAIN, smem, st>>>(g, amap, bmap, omap, rmap);
  return check_launch();
}

}  // namespace cssm
