// 32-point FFT split over 4 lanes (8 points each) and the geometry of the 32x32-plane kernels.
// lane = q + 4*g8: q = lane & 3 is the lane's index inside its FFT, g8 = lane >> 2 selects one
// of the warp's eight FFTs.
#pragma once
#include "fft.cuh"

namespace cssm {

// 4-point DFT on v[o], v[o+1], v[o+2], v[o+3]
template <bool INV, int O>
__device__ __forceinline__ void dft4(cf (&v)[8]) {
  const cf s0 = v[O] + v[O + 2], d0 = v[O] - v[O + 2];
  const cf s1 = v[O + 1] + v[O + 3], d1 = v[O + 1] - v[O + 3];
  const cf r = INV ? mk(-d1.y, d1.x) : mk(d1.y, -d1.x);     // d1 * (+i) or (-i)
  v[O] = s0 + s1; v[O + 2] = s0 - s1;
  v[O + 1] = d0 + r; v[O + 3] = d0 - r;
}

// exchange scratch: 52 cf per FFT, element (k1, j) at k1*5 + j (conflict-free scatter/gather)
constexpr int EX32_STRIDE = 52;

// Forward: in[m] = x[q + 4m]  ->  out[half*4 + k2] = X[q + 4*half + 8*k2].
// tw[k] = e^{-2 pi i q k / 32}.
__device__ __forceinline__ void fft32_fwd(cf (&v)[8], const cf (&tw)[8], cf* exg, int q) {
  dft8<false>(v);
#pragma unroll
  for (int k = 1; k < 8; ++k) v[k] = cmul(v[k], tw[k]);
#pragma unroll
  for (int k = 0; k < 8; ++k) exg[k * 5 + q] = v[k];
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j) v[h * 4 + j] = exg[(q + 4 * h) * 5 + j];
  __syncwarp();
  dft4<false, 0>(v);
  dft4<false, 4>(v);
}

// Inverse: in[half*4 + k2] = X[q + 4*half + 8*k2]  ->  out[m] = x[q + 4m] (unscaled).
__device__ __forceinline__ void fft32_inv(cf (&v)[8], const cf (&tw)[8], cf* exg, int q) {
  dft4<true, 0>(v);        // over k2 for k1 = q      -> U[q][j],   j = 0..3
  dft4<true, 4>(v);        // over k2 for k1 = q + 4  -> U[q+4][j]
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 4; ++j) exg[(q + 4 * h) * 5 + j] = v[h * 4 + j];
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = exg[k * 5 + q];      // lane j = q now holds U[k1][j], all k1
  __syncwarp();
#pragma unroll
  for (int k = 1; k < 8; ++k) v[k] = cmulc(v[k], tw[k]);  // * e^{+2 pi i q k1 / 32}
  dft8<true>(v);
}

// bin kh of a 32-point column held by lane q in register r: kh = q + 4*(r >> 2) + 8*(r & 3)
__host__ __device__ inline int r32_bin_slot(int kh) { return (((kh >> 2) & 1) << 2) | (kh >> 3); }

}  // namespace cssm
