// Dot products of a few float rows with every token of a step: a router's logits, a recurrence's gates.
#pragma once
#include "common.cuh"

#define ROW_LOGITS_MAX 256      // rows at most; the pitch of a token's results in shared memory is one more

// The logits of TOK tokens from row n0 on, left in shared memory (zs[i * (ROW_LOGITS_MAX + 1) + e]): `experts` rows of
// a float matrix (a router) and, when given, one more row (`shared_gate`) behind them.  Every warp's lanes stride over the channels
// four at a time, then a butterfly: the order of a sum depends on the sizes alone, whatever the step.
template <typename T, int TOK>
__device__ __forceinline__ void route_logits(const T* __restrict__ h, const float* __restrict__ router,
                                             const float* __restrict__ shared_gate, float* route_smem, int n_tokens, int hidden,
                                             int experts) {
  const int pitch = (hidden + 3) & ~3;
  float* xs = route_smem;
  float* zs = route_smem + TOK * pitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TOK;
  for (int i = 0; i < TOK; ++i) {
    const int n = min(n0 + i, n_tokens - 1);
    const T* row = h + (size_t)n * hidden;
    for (int c = threadIdx.x; c < hidden; c += 256) xs[i * pitch + c] = to_f32(row[c]);
  }
  __syncthreads();
  const int n_dots = experts + (shared_gate ? 1 : 0);
  const bool vec = hidden % 4 == 0 && !(((uintptr_t)router | (uintptr_t)shared_gate) & 15);
  for (int e = warp; e < n_dots; e += 8) {
    const float* w = e < experts ? router + (size_t)e * hidden : shared_gate;
    float acc[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
    if (vec) {
#pragma unroll 8
      for (int c = lane * 4; c < hidden; c += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + c);
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
          const float4 xv = *reinterpret_cast<const float4*>(xs + i * pitch + c);
          acc[i] = fmaf(wv.x, xv.x, acc[i]);
          acc[i] = fmaf(wv.y, xv.y, acc[i]);
          acc[i] = fmaf(wv.z, xv.z, acc[i]);
          acc[i] = fmaf(wv.w, xv.w, acc[i]);
        }
      }
    } else {
      for (int c = lane; c < hidden; c += 32) {
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = fmaf(w[c], xs[i * pitch + c], acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
      const float z = warp_sum(acc[i]);
      if (lane == 0) zs[i * (ROW_LOGITS_MAX + 1) + e] = z;
    }
  }
  __syncthreads();
}

