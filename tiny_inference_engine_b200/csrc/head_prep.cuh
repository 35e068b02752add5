// What is done to one query or key head of one token before attention, by one warp: RMSNorm over the head
// (src/backend/cpu/cpu_backend.cpp:118-138) and the rotate-half rotation by the token's position
// (src/backend/cpu/cpu_backend.cpp:161-193), all in float. A lane holds the VEC = head_dim / 32 neighbouring
// elements [lane * VEC, lane * VEC + VEC); an element's partner in the rotation sits in lane ^ 16. Two kernels
// share this code (the q/k norm + RoPE + append kernel and the decode attention that prepares its own heads),
// so that a head comes out the same, bit for bit, whichever of them prepared it.
#pragma once
#include "common.cuh"

namespace tie {

// VEC neighbouring elements of a head, read and written with one instruction (16 bytes at most).
template <typename T, int VEC> struct alignas(sizeof(T) * VEC > 16 ? 16 : sizeof(T) * VEC) HeadSlice {
  T v[VEC];
};

// cos at [0, half), sin at [half, 2 * half) for one position; called by the threads of a block together
// (every thread takes the indices i = first, first + step, ...), the caller synchronises before the table is read.
__device__ __forceinline__ void rotation_table(float* cs, float position, const float* __restrict__ inv_freq, int half,
                                               int first, int step) {
  for (int i = first; i < half; i += step) {
    const float angle = position * inv_freq[i];
    cs[i] = cosf(angle);
    cs[half + i] = sinf(angle);
  }
}

// x: this lane's elements of the head. w: the norm's weights (null: no norm). cs: the rotation table (null: no rotation).
template <int VEC>
__device__ __forceinline__ void prepare_head(float (&x)[VEC], const float* __restrict__ w, float eps, const float* cs, int lane) {
  constexpr int DH = 32 * VEC, HALF = DH / 2;
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < VEC; ++e) ss += x[e] * x[e];
  if (w) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(DH) + eps);
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] = (x[e] * inv) * w[lane * VEC + e];
  }
  if (cs) {
    const int i0 = (lane & 15) * VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
      const float c = cs[i0 + e], sn = cs[HALF + i0 + e];
      x[e] = lane < 16 ? x[e] * c - other * sn : x[e] * c + other * sn;
    }
  }
}

}  // namespace tie
