// Rotary angles for the kernels that rotate queries and keys.
//
// The frequency of pair j is given as a table of inverse wavelengths, inv[j] = base^(-2j/dims),
// in float32 and (for the 32-bit model path) in float64: angle = position * inv[j].  The
// bfloat16 path multiplies and takes sine and cosine in float32 (accurate sincosf); the
// 32-bit path does both in double, so that its angles are exact to float32 at any position.
#pragma once
#include "common.cuh"

#define MF_ROT_HALF 0    // channel i pairs with channel i + dims/2
#define MF_ROT_PAIRS 1   // channel 2i pairs with channel 2i + 1

__device__ __forceinline__ void rotary_cs(int pos, int j, const float* __restrict__ inv_f,
                                          const double* __restrict__ inv_d, float& c, float& s) {
  if (inv_d) {
    const double a = (double)pos * inv_d[j];
    c = (float)cos(a);
    s = (float)sin(a);
  } else {
    sincosf((float)pos * inv_f[j], &s, &c);
  }
}

// channels of pair j of a head whose first `rot` channels are rotated
__device__ __forceinline__ void rotary_pair(int layout, int rot, int j, int& a, int& b) {
  if (layout == MF_ROT_PAIRS) {
    a = 2 * j;
    b = 2 * j + 1;
  } else {
    a = j;
    b = j + (rot >> 1);
  }
}
