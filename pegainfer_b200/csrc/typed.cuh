// Element-type helpers for kernels compiled both for bf16 and for float storage: arithmetic is fp32 either way,
// a value is rounded once when it is stored.
#pragma once

#include "common.cuh"

namespace pk {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename E>
__device__ __forceinline__ E from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }

// sum_k w[k] * x[k] over a row of n elements by one warp (every lane gets the sum); x is fp32 in shared or global memory.
// bf16 rows whose length is a multiple of 8 and whose start is 16-byte aligned stream 16 bytes per lane per step.
template <typename E>
__device__ __forceinline__ float warp_dot(const E* __restrict__ w, const float* __restrict__ x, int n, int lane) {
  float acc = 0.f;
  if constexpr (sizeof(E) == 2) {
    if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
#pragma unroll 4
      for (int k = lane * 8; k < n; k += 256) {
        const uint4 v = ldg_stream(w + k);
        const float4 x0 = *reinterpret_cast<const float4*>(x + k), x1 = *reinterpret_cast<const float4*>(x + k + 4);
        acc = fmaf(bf16_lo(v.x), x0.x, acc);
        acc = fmaf(bf16_hi(v.x), x0.y, acc);
        acc = fmaf(bf16_lo(v.y), x0.z, acc);
        acc = fmaf(bf16_hi(v.y), x0.w, acc);
        acc = fmaf(bf16_lo(v.z), x1.x, acc);
        acc = fmaf(bf16_hi(v.z), x1.y, acc);
        acc = fmaf(bf16_lo(v.w), x1.z, acc);
        acc = fmaf(bf16_hi(v.w), x1.w, acc);
      }
      return warp_sum(acc);
    }
  }
  for (int k = lane; k < n; k += 32) acc = fmaf(to_f(w[k]), x[k], acc);
  return warp_sum(acc);
}

}  // namespace pk
