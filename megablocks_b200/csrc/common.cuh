// Device-side helpers shared by the sm_100a kernels.  Deliberately free of any
// PyTorch header: the .cu files see only CUDA, which keeps them fast to compile;
// tensor checks and allocation live in the .cpp glue.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "kernels.h"

namespace mb {

inline int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Index of the first entry of the ascending array `ends[0..n)` that is > v
// (the group that position v falls into when `ends` are inclusive prefix sums).
__device__ __forceinline__ int upper_bound_i32(const int* __restrict__ ends, int n, int v) {
  int lo = 0, hi = n;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (__ldg(ends + mid) <= v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Run `body` with `T` bound to the C++ type of a floating DType code.
#define MB_SWITCH_FLOAT(code, T, ...)                                        \
  switch (code) {                                                            \
    case kF32: { using T = float; __VA_ARGS__; break; }                      \
    case kF16: { using T = __half; __VA_ARGS__; break; }                     \
    case kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    default: return cudaErrorInvalidValue;                                   \
  }

#define MB_SWITCH_INT(code, T, ...)                                          \
  switch (code) {                                                            \
    case kI16: { using T = int16_t; __VA_ARGS__; break; }                    \
    case kI32: { using T = int32_t; __VA_ARGS__; break; }                    \
    case kI64: { using T = int64_t; __VA_ARGS__; break; }                    \
    default: return cudaErrorInvalidValue;                                   \
  }

}  // namespace mb
