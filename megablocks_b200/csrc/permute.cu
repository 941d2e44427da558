// Row permutation kernels for sm_100a: token order <-> expert order.
//
// Functional counterparts in the reference are the Triton row-copy kernels
// (megablocks/backend/kernels.py:34-518).  The kernels here are destination
// driven: every output row is written exactly once by one warp (payload rows,
// pad rows and rows past the last bin alike), so no output is ever pre-zeroed,
// and the reduction over the top-k copies of a token happens in registers in
// token order - deterministic, no atomics, no [tokens, k, h] staging buffer.
// Rows move as 16-byte vectors whenever the row size allows it.
#include "common.cuh"

namespace mb {

namespace {

constexpr int kWarpsPerCta = 4;

template <typename T, int VEC>
struct Pack {
  T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> load_pack(const T* p) {
  Pack<T, VEC> out;
  if constexpr (VEC * sizeof(T) == 16) {
    *reinterpret_cast<uint4*>(out.v) = *reinterpret_cast<const uint4*>(p);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out.v[i] = p[i];
  }
  return out;
}

template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, VEC>& in) {
  if constexpr (VEC * sizeof(T) == 16) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(in.v);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = in.v[i];
  }
}

// out[r] for every row r of the expert-ordered buffer:
//   e = group of r in padded_bins, off = r - padded_start(e);
//   off < count(e): x[indices[start(e) + off] / top_k] (* weight), else zero.
template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ indices, const T* __restrict__ weights, const int* __restrict__ bins,
                   const int* __restrict__ padded_bins, int num_bins, int top_k, int64_t out_rows, int cols,
                   T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t r = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (r >= out_rows) return;
  int src_token = -1;
  float scale = 1.f;
  const int e = upper_bound_i32(padded_bins, num_bins, static_cast<int>(r));
  if (e < num_bins) {
    const int pstart = e ? __ldg(padded_bins + e - 1) : 0;
    const int start = e ? __ldg(bins + e - 1) : 0;
    const int count = __ldg(bins + e) - start;
    const int off = static_cast<int>(r) - pstart;
    if (off < count) {
      const int copy = __ldg(indices + start + off);
      src_token = copy / top_k;
      if (weights != nullptr) scale = to_float(weights[copy]);
    }
  }
  T* dst = out + r * cols;
  if (src_token < 0) {
    Pack<T, VEC> z;
#pragma unroll
    for (int i = 0; i < VEC; ++i) z.v[i] = from_float<T>(0.f);
    for (int c = lane * VEC; c < cols; c += 32 * VEC) store_pack<T, VEC>(dst + c, z);
    return;
  }
  const T* src = x + int64_t(src_token) * cols;
  if (weights == nullptr) {
    // Four vector loads in flight per lane before the first store.
    for (int c0 = lane * VEC; c0 < cols; c0 += 4 * 32 * VEC) {
      Pack<T, VEC> p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + j * 32 * VEC < cols) p[j] = load_pack<T, VEC>(src + c0 + j * 32 * VEC);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + j * 32 * VEC < cols) store_pack<T, VEC>(dst + c0 + j * 32 * VEC, p[j]);
    }
  } else {
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> p = load_pack<T, VEC>(src + c);
#pragma unroll
      for (int i = 0; i < VEC; ++i) p.v[i] = from_float<T>(to_float(p.v[i]) * scale);
      store_pack<T, VEC>(dst + c, p);
    }
  }
}

// inverse[copy] = row of that copy in the expert-ordered buffer (or -1 when dropped).
// capacity < 0: padded layout (row = padded_start(e) + off); capacity >= 0: binned
// layout (row = e * capacity + off, dropped when off >= capacity).
__global__ void inverse_map_kernel(const int* __restrict__ indices, const int* __restrict__ bins,
                                   const int* __restrict__ padded_bins, int num_bins, int n, int capacity,
                                   int* __restrict__ inverse) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = upper_bound_i32(bins, num_bins, i);
  if (e >= num_bins) {            // a position past the last bin: its copy belongs to no expert
    inverse[__ldg(indices + i)] = -1;
    return;
  }
  const int off = i - (e ? __ldg(bins + e - 1) : 0);
  int row;
  if (capacity < 0) row = (e ? __ldg(padded_bins + e - 1) : 0) + off;
  else row = off < capacity ? e * capacity + off : -1;
  inverse[__ldg(indices + i)] = row;
}

// out[t] = sum_s weight[t*k+s] * x[inverse[t*k+s]]  (fp32 accumulate, one rounding).
template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
combine_rows_kernel(const T* __restrict__ x, const int* __restrict__ inverse, const T* __restrict__ weights,
                    int top_k, int64_t tokens, int cols, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (t >= tokens) return;
  T* dst = out + t * cols;
  if (top_k == 1) {
    const int row = __ldg(inverse + t);
    const float w = (weights != nullptr) ? to_float(weights[t]) : 1.f;
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> p;
      if (row >= 0) {
        p = load_pack<T, VEC>(x + int64_t(row) * cols + c);
        if (weights != nullptr) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) p.v[i] = from_float<T>(to_float(p.v[i]) * w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) p.v[i] = from_float<T>(0.f);
      }
      store_pack<T, VEC>(dst + c, p);
    }
    return;
  }
  for (int c = lane * VEC; c < cols; c += 32 * VEC) {
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int s = 0; s < top_k; ++s) {
      const int64_t copy = t * top_k + s;
      const int row = __ldg(inverse + copy);
      if (row < 0) continue;
      const float w = (weights != nullptr) ? to_float(weights[copy]) : 1.f;
      Pack<T, VEC> p = load_pack<T, VEC>(x + int64_t(row) * cols + c);
      // Each product is rounded to T before the sum, as when the k scaled copies
      // are first stored and then added.
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += to_float(from_float<T>(to_float(p.v[i]) * w));
    }
    Pack<T, VEC> o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = from_float<T>(acc[i]);
    store_pack<T, VEC>(dst + c, o);
  }
}

// wgrad[copy] = <x[row(copy)], grad[copy / top_k]>, one warp per copy.  VEC > 1: both rows are read
// in 16-byte pieces (rows of a multiple of 16 bytes at 16-byte aligned bases).
template <typename T, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
wgrad_kernel(const T* __restrict__ x, const T* __restrict__ grad, const int* __restrict__ inverse, int top_k,
             int64_t copies, int cols, T* __restrict__ wgrad) {
  const int lane = threadIdx.x & 31;
  const int64_t copy = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (copy >= copies) return;
  const int row = __ldg(inverse + copy);
  float acc = 0.f;
  if (row >= 0) {
    const T* a = x + int64_t(row) * cols;
    const T* b = grad + (copy / top_k) * cols;
    if constexpr (VEC > 1) {
      float acc2 = 0.f;
      for (int c = lane * VEC; c < cols; c += 32 * VEC) {
        const Pack<T, VEC> pa = load_pack<T, VEC>(a + c), pb = load_pack<T, VEC>(b + c);
#pragma unroll
        for (int k = 0; k < VEC; k += 2) {
          acc = fmaf(to_float(pa.v[k]), to_float(pb.v[k]), acc);
          acc2 = fmaf(to_float(pa.v[k + 1]), to_float(pb.v[k + 1]), acc2);
        }
      }
      acc += acc2;
    } else {
      for (int c = lane; c < cols; c += 32) acc += to_float(a[c]) * to_float(b[c]);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) wgrad[copy] = from_float<T>(acc);
}

template <typename T>
int vec_width(int64_t cols, const void* a, const void* b) {
  constexpr int full = 16 / sizeof(T);
  const bool aligned = (reinterpret_cast<uintptr_t>(a) % 16 == 0) && (reinterpret_cast<uintptr_t>(b) % 16 == 0);
  return (aligned && cols % full == 0) ? full : 1;
}

}  // namespace

cudaError_t gather_rows(DType type, const void* x, const int* indices, const void* weights, const int* bins,
                        const int* padded_bins, int num_bins, int top_k, int64_t out_rows, int cols, void* out,
                        cudaStream_t stream) {
  const int grid = ceil_div(out_rows, kWarpsPerCta);
  MB_SWITCH_FLOAT(type, T, {
    constexpr int kFull = 16 / sizeof(T);
    if (vec_width<T>(cols, x, out) > 1) {
      gather_rows_kernel<T, kFull><<<grid, kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), indices, static_cast<const T*>(weights), bins, padded_bins, num_bins, top_k,
          out_rows, cols, static_cast<T*>(out));
    } else {
      gather_rows_kernel<T, 1><<<grid, kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), indices, static_cast<const T*>(weights), bins, padded_bins, num_bins, top_k,
          out_rows, cols, static_cast<T*>(out));
    }
  })
  return cudaGetLastError();
}

cudaError_t inverse_map(const int* indices, const int* bins, const int* padded_bins, int num_bins, int n,
                        int capacity, int* inverse, cudaStream_t stream) {
  inverse_map_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(indices, bins, padded_bins, num_bins, n, capacity,
                                                          inverse);
  return cudaGetLastError();
}

cudaError_t combine_rows(DType type, const void* x, const int* inverse, const void* weights, int top_k,
                         int64_t tokens, int cols, void* out, cudaStream_t stream) {
  const int grid = ceil_div(tokens, kWarpsPerCta);
  MB_SWITCH_FLOAT(type, T, {
    constexpr int kFull = 16 / sizeof(T);
    if (vec_width<T>(cols, x, out) > 1) {
      combine_rows_kernel<T, kFull><<<grid, kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), inverse, static_cast<const T*>(weights), top_k, tokens, cols,
          static_cast<T*>(out));
    } else {
      combine_rows_kernel<T, 1><<<grid, kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), inverse, static_cast<const T*>(weights), top_k, tokens, cols,
          static_cast<T*>(out));
    }
  })
  return cudaGetLastError();
}

cudaError_t scatter_wgrad(DType type, const void* x, const void* grad, const int* inverse, int top_k,
                          int64_t copies, int cols, void* wgrad, cudaStream_t stream) {
  MB_SWITCH_FLOAT(type, T, {
    constexpr int kFull = 16 / sizeof(T);
    if (vec_width<T>(cols, x, grad) > 1) {
      wgrad_kernel<T, kFull><<<ceil_div(copies, kWarpsPerCta), kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), static_cast<const T*>(grad), inverse, top_k, copies, cols,
          static_cast<T*>(wgrad));
    } else {
      wgrad_kernel<T, 1><<<ceil_div(copies, kWarpsPerCta), kWarpsPerCta * 32, 0, stream>>>(
          static_cast<const T*>(x), static_cast<const T*>(grad), inverse, top_k, copies, cols,
          static_cast<T*>(wgrad));
    }
  })
  return cudaGetLastError();
}

}  // namespace mb
