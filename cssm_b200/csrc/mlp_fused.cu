// Fused MLP of the stage-0 ConvBlock of CSSM-SHViT (Mlp in src/models/shvit.py:165-180 after the
// block's LayerNorm: fc1 64 -> 256, GELU, fc2 256 -> 64, plus the residual):
//   out[m, :] = res[m, :] + W2^T gelu(W1^T a[m, :] + b1) + b2
// as ONE kernel, so that the hidden tensor (M x 256 bf16: four times the block's input) never leaves
// the SM: HBM sees a, res and out.  Persistent, one CTA per SM, 608 threads, warp-specialised:
//   warp 0      TMA producer: both weight matrices once (64 KB, resident in shared memory), then the
//               128-row input tile of every M tile into a 4-stage ring;
//   warps 1, 2  MMA issuers, one per epilogue half (a half owns every other tile end to end):
//               fc1 in four 64-column chunks alternating between the half's two TMEM accumulators
//               (tcgen05.mma.kind::f16, M128 x N64 x K16), fc2 (K = 256, one K block per chunk) from the
//               hidden chunks the epilogue wrote back to shared memory as a K-major operand;
//   warps 3-18  epilogue, two halves of eight warps (two per TMEM lane quadrant, one for each 32
//               columns of a chunk; four warps per scheduler hide the GELU latency): tcgen05.ld of a
//               hidden chunk, bias, GELU, bf16 -> one of the half's two 128 x 64 hidden buffers in the
//               128-byte swizzle; after fc2: bias, residual (fetched by TMA into the staging box during
//               the tile), bf16, TMA tensor store.  The fc2 accumulator of a tile is drained after chunk 0
//               of the half's next tile, when its last fc2 has long finished.
// The warps hand over through mbarriers only (no named barrier, no block barrier inside the loop); every
// wait is bounded, and on expiry the kernel records an error code (cssm_device_error) and winds down.
// No multicast, no cluster.
#include <cuda.h>
#include <cuda_bf16.h>
#include <string.h>
#include "kernels.cuh"
#include "tc05.cuh"
#include "bf16_ops.cuh"

namespace cssm {

__device__ int g_mlp_error = 0;

constexpr int MF_THREADS = 608, MF_C = 64, MF_HD = 256, MF_NS = 4;
constexpr uint32_t MF_W1_BYTES = 2u * 16384u;          // two chunks of 128 hidden rows x 64 k
constexpr uint32_t MF_W2_BYTES = 4u * 8192u;           // four K blocks of 64 output rows x 64 k
constexpr uint32_t MF_T_BYTES = 16384u;                // 128 rows x 64 k
constexpr uint32_t MF_HS_BYTES = 32768u;               // per half: two K blocks of 128 rows x 64 k
constexpr uint32_t MF_OUT_BYTES = 16384u;              // per half: one 128 x 64 staging box
constexpr uint32_t MF_SMEM = MF_W1_BYTES + MF_W2_BYTES + MF_NS * MF_T_BYTES + 2 * MF_HS_BYTES + 2 * MF_OUT_BYTES;

__device__ __forceinline__ uint32_t mf_idesc(uint32_t M, uint32_t N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);   // f32 acc, bf16 A and B
}
__device__ __forceinline__ void mf_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

struct MlpFusedArgs {
  int M;
  const float* b1;           // (256)
  const float* b2;           // (64)
};

__global__ void __launch_bounds__(MF_THREADS, 1)
mlp_fused_kernel(const MlpFusedArgs g, const __grid_constant__ CUtensorMap amap,
                 const __grid_constant__ CUtensorMap w1map, const __grid_constant__ CUtensorMap w2map,
                 const __grid_constant__ CUtensorMap rmap, const __grid_constant__ CUtensorMap omap) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* w1s = smem;
  unsigned char* w2s = w1s + MF_W1_BYTES;
  unsigned char* ts = w2s + MF_W2_BYTES;
  unsigned char* hs = ts + MF_NS * MF_T_BYTES;
  unsigned char* outs = hs + 2 * MF_HS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(outs + 2 * MF_OUT_BYTES);
  uint64_t* tfull = bars;            // [MF_NS]
  uint64_t* tempty = bars + 4;       // [MF_NS]
  uint64_t* wfull = bars + 8;        // [1]
  uint64_t* acc1full = bars + 9;     // [half][2]: fc1 accumulator b of the half complete
  uint64_t* acc1empty = bars + 13;   // [half][2]
  uint64_t* hsfull = bars + 17;      // [half][2]: hidden buffer b written
  uint64_t* acc2full = bars + 21;    // [2] per half
  uint64_t* acc2empty = bars + 23;   // [2]
  uint64_t* resfull = bars + 25;     // [2]
  uint64_t* done = bars + 27;        // [2] per MMA warp
  uint64_t* stfull = bars + 29;      // [2] per half: the output box is complete in the staging slot
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 31);
  float* b1s = reinterpret_cast<float*>(bars + 64);      // both bias vectors, read by every epilogue warp
  float* b2s = b1s + MF_HD;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_tiles = (g.M + 127) / 128;
  const uint32_t sbase = tc::smem_u32(smem);

  if (tid == 0) {
    for (int s = 0; s < MF_NS; ++s) { tc::mbar_init(&tfull[s], 1); tc::mbar_init(&tempty[s], 1); }
    tc::mbar_init(wfull, 1);
    for (int h = 0; h < 2; ++h) {
      for (int b = 0; b < 2; ++b) {
        tc::mbar_init(&acc1full[2 * h + b], 1);
        tc::mbar_init(&acc1empty[2 * h + b], 8);      // one lane per warp of the half
        tc::mbar_init(&hsfull[2 * h + b], 8);
      }
      tc::mbar_init(&acc2full[h], 1);
      tc::mbar_init(&acc2empty[h], 8);
      tc::mbar_init(&resfull[h], 1);
      tc::mbar_init(&done[h], 1);
      tc::mbar_init(&stfull[h], 8);
    }
    tc::fence_mbar_init();
  }
  for (int i = tid; i < MF_HD + MF_C; i += MF_THREADS) b1s[i] = i < MF_HD ? g.b1[i] : g.b2[i - MF_HD];
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, 512);
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
      tc::mbar_expect_tx(wfull, MF_W1_BYTES + MF_W2_BYTES);
      tc::tma_load_2d(w1s, &w1map, 0, 0, wfull);
      tc::tma_load_2d(w1s + 16384, &w1map, 0, 128, wfull);
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) tc::tma_load_2d(w2s + kb * 8192, &w2map, kb * 64, 0, wfull);
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const int s = it % MF_NS;
        if (!tc::mbar_wait(&tempty[s], ((it / MF_NS) & 1) ^ 1)) { atomicExch(&g_mlp_error, 1); bad = true; break; }
        tc::mbar_expect_tx(&tfull[s], MF_T_BYTES);
        tc::tma_load_2d(ts + s * MF_T_BYTES, &amap, 0, tile * 128, &tfull[s]);
      }
    }
    __syncwarp();
  } else if (warp < 3) {
    // ================================ MMA issuers ================================
    const int half = warp - 1;
    if (lane == 0) {
      const uint32_t acc1 = tmem_base + (uint32_t)half * 192u, acc2 = acc1 + 128u;   // acc1: two 64-column buffers
      const uint32_t id = mf_idesc(128, 64);
      const uint32_t hs_a = sbase + (uint32_t)(hs - smem) + (uint32_t)half * MF_HS_BYTES;
      const uint32_t w1_a = sbase + (uint32_t)(w1s - smem), w2_a = sbase + (uint32_t)(w2s - smem);
      if (!tc::mbar_wait(wfull, 0)) { atomicExch(&g_mlp_error, 2); bad = true; }
      int it = 0, j = 0;                               // it: CTA-local tile index; j: tiles of this half
      // fc2 over hidden chunk ch (64 columns = one K block) of the half's j-th tile
      auto fc2_chunk = [&](int ch) -> bool {
        const int b = ch & 1, nb = (4 * j + ch) >> 1;          // nb-th use of hidden buffer b
        if (ch == 0 && !tc::mbar_wait(&acc2empty[half], (j & 1) ^ 1)) { atomicExch(&g_mlp_error, 5); return false; }
        if (!tc::mbar_wait(&hsfull[2 * half + b], nb & 1)) { atomicExch(&g_mlp_error, 6); return false; }
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mf_mma(acc2, tc::make_desc_sw128(hs_a + b * 16384u + ks * 32u),
                 tc::make_desc_sw128(w2_a + ch * 8192u + ks * 32u), id, (ch | ks) ? 1u : 0u);
        return true;
      };
      for (int tile = blockIdx.x; tile < num_tiles && !bad; tile += gridDim.x, ++it) {
        if ((it & 1) != half) continue;
        const int s = it % MF_NS;
        const uint32_t t_a = sbase + (uint32_t)(ts - smem) + (uint32_t)s * MF_T_BYTES;
        if (!tc::mbar_wait(&tfull[s], (it / MF_NS) & 1)) { atomicExch(&g_mlp_error, 3); bad = true; break; }
        // fc1 in four chunks of 64 hidden columns through two accumulators; the fc2 of a chunk is
        // issued one chunk later, while the epilogue works on the next accumulator
        for (int ch = 0; ch < 4 && !bad; ++ch) {
          const int b = ch & 1, nb = (4 * j + ch) >> 1;
          if (!tc::mbar_wait(&acc1empty[2 * half + b], (nb & 1) ^ 1)) { atomicExch(&g_mlp_error, 4); bad = true; break; }
          tc::fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mf_mma(acc1 + b * 64u, tc::make_desc_sw128(t_a + ks * 32u),
                   tc::make_desc_sw128(w1_a + ch * 8192u + ks * 32u), id, ks ? 1u : 0u);
          tc::commit(&acc1full[2 * half + b]);
          if (ch == 3) tc::commit(&tempty[s]);         // the input tile has been read by all chunks
          if (ch > 0 && !fc2_chunk(ch - 1)) { bad = true; break; }
        }
        if (bad) break;
        if (!fc2_chunk(3)) { bad = true; break; }
        tc::commit(&acc2full[half]);
        ++j;
      }
      // nothing of this thread's tensor work may be in flight when TMEM is freed
      tc::commit(&done[half]);
      if (!tc::mbar_wait(&done[half], 0) && !bad) atomicExch(&g_mlp_error, 8);
    }
    __syncwarp();
  } else {
    // ================================ epilogue ================================
    // eight warps per half: two per TMEM lane quadrant (warp id mod 4), one for each 32-column part
    // of a 64-column chunk -- four warps per scheduler, which is what hides the GELU latency
    const int q = warp & 3;
    const int half = (warp - 3) >> 3;
    const int sub = ((warp - 3) >> 2) & 1;
    const int row = q * 32 + lane;
    const bool issuer = ((warp - 3) & 7) == 0 && lane == 0;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)half * 192u;
    unsigned char* hsh = hs + half * MF_HS_BYTES;
    unsigned char* stg = outs + half * MF_OUT_BYTES;
    int it = 0, j = 0;
    bool live = true;
    // every wait is bounded and its outcome is made uniform over the warp (the TMEM loads that follow
    // want the warp converged); a warp that gives up leaves its loop, the others run into their own limits
    auto wok = [](bool ok) { return __all_sync(0xffffffffu, ok) != 0; };
    uint32_t ra[32];
    // one 64-column chunk of the hidden layer of the half's j-th tile: bias, GELU, bf16 -> hidden buffer
    auto hidden_chunk = [&](int ch) -> bool {
      const int b = ch & 1, nb = (4 * j + ch) >> 1;          // nb-th use of accumulator / hidden buffer b
      if (!wok(tc::mbar_wait_spin(&acc1full[2 * half + b], nb & 1))) { atomicExch(&g_mlp_error, 9); return false; }
      tc::fence_after_sync();
      // (the fc2 that read the previous contents of this hidden buffer was issued before this chunk's
      // fc1, and a commit covers everything its thread issued before it: the buffer is free)
      unsigned char* kb = hsh + b * 16384u;
      float v[32];
      tc::ld_32x32b_x32(tlane + b * 64 + sub * 32, ra);
      tc::wait_ld();
      const float4* bp = reinterpret_cast<const float4*>(b1s + ch * 64 + sub * 32);
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4) {
        const float4 b4 = bp[jj >> 2];
        upk2(add2(pk2(__uint_as_float(ra[jj]), __uint_as_float(ra[jj + 1])), pk2(b4.x, b4.y)), v[jj], v[jj + 1]);
        upk2(add2(pk2(__uint_as_float(ra[jj + 2]), __uint_as_float(ra[jj + 3])), pk2(b4.z, b4.w)), v[jj + 2], v[jj + 3]);
      }
#pragma unroll
      for (int jj = 0; jj < 32; jj += 2) gelu_tanh_x2(v[jj], v[jj + 1]);
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        const float f[8] = {v[j4 * 8], v[j4 * 8 + 1], v[j4 * 8 + 2], v[j4 * 8 + 3],
                            v[j4 * 8 + 4], v[j4 * 8 + 5], v[j4 * 8 + 6], v[j4 * 8 + 7]};
        *reinterpret_cast<uint4*>(kb + tc::sw128_offset(row, sub * 4 + j4)) = pack8(f);
      }
      // accumulator read, hidden chunk written: hand both to the MMA warp
      tc::fence_before_sync();
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) { tc::mbar_arrive(&acc1empty[2 * half + b]); tc::mbar_arrive(&hsfull[2 * half + b]); }
      return true;
    };
    // the fc2 accumulator of the half's jp-th tile (rows m0p..): bias, residual, bf16, store
    auto drain = [&](int m0p, int jp) -> bool {
      if (!wok(tc::mbar_wait_spin(&acc2full[half], jp & 1))) { atomicExch(&g_mlp_error, 11); return false; }
      tc::fence_after_sync();
      if (!wok(tc::mbar_wait_spin(&resfull[half], jp & 1))) { atomicExch(&g_mlp_error, 12); return false; }
      uint4 pk[4];
      {
        float v[32];
        tc::ld_32x32b_x32(tlane + 128 + sub * 32, ra);
        tc::wait_ld();
        const float4* bp = reinterpret_cast<const float4*>(b2s + sub * 32);
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          const float4 b4 = bp[jj >> 2];
          v[jj] = __uint_as_float(ra[jj]) + b4.x; v[jj + 1] = __uint_as_float(ra[jj + 1]) + b4.y;
          v[jj + 2] = __uint_as_float(ra[jj + 2]) + b4.z; v[jj + 3] = __uint_as_float(ra[jj + 3]) + b4.w;
        }
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          float f[8];
          unpack8(*reinterpret_cast<const uint4*>(stg + tc::sw128_offset(row, sub * 4 + j4)), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] += v[j4 * 8 + e];
          pk[j4] = pack8(f);
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc2empty[half]);
#pragma unroll
      for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(stg + tc::sw128_offset(row, sub * 4 + c)) = pk[c];
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&stfull[half]);
      bool ok = true;
      if (issuer) {
        // all eight warps of the half have written their part of the box (a bounded wait each, so
        // that a warp that gave up cannot leave the others behind a barrier)
        if (tc::mbar_wait_spin(&stfull[half], jp & 1)) {
          tc::tma_store_2d(&omap, stg, 0, m0p);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        } else {
          atomicExch(&g_mlp_error, 13);
          ok = false;
        }
      }
      return wok(ok);
    };
    // Order per tile: chunk 0, the previous tile's fc2 accumulator (its last fc2 has long finished by
    // then, so nothing waits for the tensor pipe), chunk 1, the residual fetch, chunks 2 and 3.
    int m0_prev = 0;
    for (int tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x, ++it) {
      if ((it & 1) != half) continue;
      const int m0 = tile * 128;
      live = hidden_chunk(0);
      if (live && j > 0) live = drain(m0_prev, j - 1);
      if (live) live = hidden_chunk(1);
      if (!live) break;
      if (issuer) {
        // the previous tile's store has read the staging box: fetch this tile's residual into it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        tc::mbar_expect_tx(&resfull[half], MF_OUT_BYTES);
        tc::tma_load_2d(stg, &rmap, 0, m0, &resfull[half]);
      }
      __syncwarp();
      live = hidden_chunk(2);
      if (live) live = hidden_chunk(3);
      m0_prev = m0;
      ++j;
    }
    if (live && j > 0) drain(m0_prev, j - 1);
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  // error path only: give copies that may still be in flight a bounded time to land
  if (bad)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*MfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MfEncodeFn mf_encode_fn() {
  static MfEncodeFn fn = []() -> MfEncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<MfEncodeFn>(p);
  }();
  return fn;
}
// bf16 matrix [rows][cols] with row stride ld elements -> boxes of 64 columns x box_rows rows, 128-byte swizzle
static bool mf_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  MfEncodeFn enc = mf_encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {64, box_rows}, es[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool mlp_fused_supported(int C, int Hd) { return C == MF_C && Hd == MF_HD; }

int read_mlp_error(int* out, int clear) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_mlp_error, sizeof(int));
  if (e == cudaSuccess && clear && *out != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_mlp_error, &zero, sizeof(int));
  }
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  return CSSM_OK;
}

// a (M, 64) bf16; w1t (256, 64) and w2t (64, 256) bf16 K-major (as launch_pack_wt writes them, row
// strides ld1 / ld2); b1 (256), b2 (64) float32; res, out (M, 64) bf16.
int launch_mlp_fused(const __nv_bfloat16* a, int M, const __nv_bfloat16* w1t, int ld1, const float* b1,
                     const __nv_bfloat16* w2t, int ld2, const float* b2, const __nv_bfloat16* res,
                     __nv_bfloat16* out, cudaStream_t st) {
  if (M <= 0) return CSSM_ERR_DIMS;
  if (!a || !w1t || !b1 || !w2t || !b2 || !res || !out) return CSSM_ERR_NULL;
  if (!aligned16(a) || !aligned16(w1t) || !aligned16(w2t) || !aligned16(res) || !aligned16(out) ||
      !aligned16(b1) || !aligned16(b2))
    return CSSM_ERR_ALIGN;
  if (ld1 < MF_C || ld2 < MF_HD || ld1 % 8 != 0 || ld2 % 8 != 0) return CSSM_ERR_UNSUPPORTED;
  CUtensorMap amap, w1map, w2map, rmap, omap;
  if (!mf_map(&amap, a, (uint64_t)M, MF_C, MF_C, 128) || !mf_map(&w1map, w1t, MF_HD, MF_C, (uint64_t)ld1, 128) ||
      !mf_map(&w2map, w2t, MF_C, MF_HD, (uint64_t)ld2, 64) || !mf_map(&rmap, res, (uint64_t)M, MF_C, MF_C, 128) ||
      !mf_map(&omap, out, (uint64_t)M, MF_C, MF_C, 128))
    return CSSM_ERR_CUDA;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t smem = MF_SMEM + 512 + (MF_HD + MF_C) * sizeof(float) + 1024;
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(mlp_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { set_cuda_error(e); return CSSM_ERR_CUDA; }
  const int tiles = (M + 127) / 128;
  MlpFusedArgs g;
  g.M = M; g.b1 = b1; g.b2 = b2;
  mlp_fused_kernel<<<tiles < sms ? tiles : sms, MF_THREADS, smem, st>>>(g, amap, w1map, w2map, rmap, omap);
  return check_launch();
}

}  // namespace cssm
