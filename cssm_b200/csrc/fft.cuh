// In-register radix-8 / radix-4 DFT butterflies and the 8x8 split of a 64-point FFT
// over 8 lanes with one shared-memory exchange.
#pragma once
#include "common.cuh"

namespace cssm {

// 8-point DFT, natural order in and out.  INV=false: e^{-2 pi i nk/8}; INV=true: e^{+...}.
template <bool INV>
__device__ __forceinline__ void dft8(cf (&a)[8]) {
  constexpr float R = 0.70710678118654752440f;
  cf b0 = a[0] + a[4], b4 = a[0] - a[4];
  cf b1 = a[1] + a[5], b5 = a[1] - a[5];
  cf b2 = a[2] + a[6], b6 = a[2] - a[6];
  cf b3 = a[3] + a[7], b7 = a[3] - a[7];
  if (!INV) {
    b5 = mk(R * (b5.x + b5.y), R * (b5.y - b5.x));   // * e^{-i pi/4}
    b6 = mk(b6.y, -b6.x);                            // * -i
    b7 = mk(R * (b7.y - b7.x), -R * (b7.x + b7.y));  // * e^{-3i pi/4}
  } else {
    b5 = mk(R * (b5.x - b5.y), R * (b5.x + b5.y));   // * e^{+i pi/4}
    b6 = mk(-b6.y, b6.x);                            // * +i
    b7 = mk(-R * (b7.x + b7.y), R * (b7.x - b7.y));  // * e^{+3i pi/4}
  }
  cf c0 = b0 + b2, c2 = b0 - b2, c1 = b1 + b3, d3 = b1 - b3;
  cf c4 = b4 + b6, c6 = b4 - b6, c5 = b5 + b7, d7 = b5 - b7;
  cf c3 = INV ? mk(-d3.y, d3.x) : mk(d3.y, -d3.x);
  cf c7 = INV ? mk(-d7.y, d7.x) : mk(d7.y, -d7.x);
  a[0] = c0 + c1; a[4] = c0 - c1;
  a[2] = c2 + c3; a[6] = c2 - c3;
  a[1] = c4 + c5; a[5] = c4 - c5;
  a[3] = c6 + c7; a[7] = c6 - c7;
}

// Geometry of one 64-point FFT shared by the 8 lanes {sub + 4*a : a = 0..7} of a warp
// (sub = lane & 3 selects one of the warp's four FFTs, a = lane >> 2 is the lane's index
// inside it).  Exchange scratch: one 76-element cf region per FFT, element (k, j) at
// k*9 + j; with these strides both the scatter and the gather are bank-conflict free for
// 64-bit accesses.
constexpr int EX_GROUP_STRIDE = 76;

// Forward: in[m] = x[a + 8m]  ->  out[k2] = X[a + 8*k2].   tw[k] = e^{-2 pi i a k / 64}.
// Inverse: in[m] = X[a + 8m]  ->  out[n1] = x[a + 8*n1] (unscaled), same tw (conjugated).
template <bool INV>
__device__ __forceinline__ void fft64_lane8(cf (&v)[8], const cf (&tw)[8], cf* exg, int a) {
  dft8<INV>(v);
#pragma unroll
  for (int k = 1; k < 8; ++k) v[k] = INV ? cmulc(v[k], tw[k]) : cmul(v[k], tw[k]);
#pragma unroll
  for (int k = 0; k < 8; ++k) exg[k * 9 + a] = v[k];
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = exg[a * 9 + j];
  __syncwarp();
  dft8<INV>(v);
}

}  // namespace cssm
