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

}  // namespace pk
