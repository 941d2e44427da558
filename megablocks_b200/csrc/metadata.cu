// Integer metadata kernels for sm_100a: stable radix / counting sort, histogram,
// row prefix sums, block-diagonal topology, replicate, and the fused route plan.
//
// Functional counterparts in the reference are CUB library calls and two small
// kernels (csrc/sort.h:19-86, histogram.h:19-81, cumsum.h:65-156, indices.h:14-93,
// replicate.h:21-206).  These kernels are written from scratch around one
// observation: every key space here is tiny (expert ids, <= 1024 values, or one
// 8-bit digit), so a sort is a histogram, a scan and one stable placement pass,
// and the histogram / prefix sums the caller wants next fall out of the same passes.
#include <atomic>

#include "common.cuh"
#include "route_plan_noalloc.h"

#include <cstdio>

namespace mb {

namespace {

constexpr int kSortWarps = 8;            // warps per CTA in the sort passes
constexpr int kSortThreads = kSortWarps * 32;

// Elements handled by one warp.  Stability needs each warp to own one contiguous
// chunk and walk it in order.
__host__ __device__ inline int warp_chunk(int64_t n) {
  if (n <= (1 << 16)) return 512;
  if (n <= (1 << 20)) return 2048;
  return 8192;
}

template <typename K>
__device__ __forceinline__ int digit_of(K key, int shift, int bits, bool flip_sign) {
  using U = typename std::make_unsigned<K>::type;
  U u = static_cast<U>(key);
  if (flip_sign) u ^= (U(1) << (sizeof(K) * 8 - 1));
  return static_cast<int>((u >> shift) & ((U(1) << bits) - 1));
}

// Pass 1: per-warp digit histograms.  partial is [nbins][num_chunks] so that the
// per-bin scan of pass 2 reads contiguously.
template <typename K>
__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const K* __restrict__ keys, int64_t n, int shift, int bits, bool flip_sign, int chunk,
                 int num_chunks, int* __restrict__ partial) {
  extern __shared__ int smem[];
  const int nbins = 1 << bits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* hist = smem + warp * nbins;
  for (int b = lane; b < nbins; b += 32) hist[b] = 0;
  __syncwarp();
  const int c = blockIdx.x * kSortWarps + warp;
  if (c < num_chunks) {
    const int64_t begin = int64_t(c) * chunk;
    const int64_t end = min(begin + chunk, n);
    for (int64_t i = begin + lane; i < end; i += 32) atomicAdd(&hist[digit_of(keys[i], shift, bits, flip_sign)], 1);
    __syncwarp();
    for (int b = lane; b < nbins; b += 32) partial[int64_t(b) * num_chunks + c] = hist[b];
  }
}

// Pass 2: one CTA per bin turns that bin's per-chunk counts into an exclusive
// prefix over chunks and records the bin total.
__global__ void __launch_bounds__(256) sort_scan_kernel(int* __restrict__ partial, int num_chunks,
                                                        int* __restrict__ totals) {
  __shared__ int warp_sums[8];
  __shared__ int carry_s;
  int* row = partial + int64_t(blockIdx.x) * num_chunks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < num_chunks; base += 256) {
    const int i = base + threadIdx.x;
    const int v = i < num_chunks ? row[i] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int warp_off = 0;
    for (int w = 0; w < warp; ++w) warp_off += warp_sums[w];
    const int carry = carry_s;
    if (i < num_chunks) row[i] = carry + warp_off + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = carry + warp_off + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry_s;
}

// Exclusive scan of up to 1024 bin totals by one CTA of kSortThreads threads.
// Leaves bin_base[b] = sum of totals of bins < b in shared memory.
__device__ void block_scan_totals(const int* __restrict__ totals, int nbins, int* bin_base, int* scratch) {
  // Each thread owns up to 4 consecutive bins (256 threads x 4 = 1024).
  const int per = (nbins + kSortThreads - 1) / kSortThreads;
  const int first = threadIdx.x * per;
  int local[4] = {0, 0, 0, 0};
  int sum = 0;
  for (int j = 0; j < per; ++j) {
    const int b = first + j;
    local[j] = b < nbins ? totals[b] : 0;
    sum += local[j];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  int off = incl - sum;
  for (int w = 0; w < warp; ++w) off += scratch[w];
  for (int j = 0; j < per; ++j) {
    const int b = first + j;
    if (b < nbins) bin_base[b] = off;
    off += local[j];
  }
  __syncthreads();
}

// Pass 3: stable placement.  Optionally (route plan) CTA 0 also writes the
// per-bin totals, their inclusive prefix sums and the block-padded prefix sums.
template <typename K, typename V>
__global__ void __launch_bounds__(kSortThreads)
sort_place_kernel(const K* __restrict__ keys, const V* __restrict__ vals_in, int64_t n, int shift, int bits,
                  bool flip_sign, int chunk, int num_chunks, const int* __restrict__ partial,
                  const int* __restrict__ totals, K* __restrict__ keys_out, V* __restrict__ vals_out,
                  int* __restrict__ tpe_out, int* __restrict__ bins_out, int* __restrict__ padded_bins_out,
                  int num_real_bins, int block) {
  extern __shared__ int smem[];
  const int nbins = 1 << bits;
  int* bin_base = smem;                       // [nbins]
  int* scratch = smem + nbins;                // [8]
  int* cursors = smem + nbins + 8;            // [kSortWarps][nbins]
  block_scan_totals(totals, nbins, bin_base, scratch);

  if (blockIdx.x == 0 && tpe_out != nullptr) {
    // Padded prefix sums need their own scan; nbins is small, so one thread per
    // bin sums its predecessors' padded sizes.
    for (int b = threadIdx.x; b < num_real_bins; b += kSortThreads) {
      const int t = totals[b];
      tpe_out[b] = t;
      bins_out[b] = bin_base[b] + t;
    }
    for (int b = threadIdx.x; b < num_real_bins; b += kSortThreads) {
      int acc = 0;
      for (int j = 0; j <= b; ++j) acc += ((totals[j] + block - 1) / block) * block;
      padded_bins_out[b] = acc;
    }
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * kSortWarps + warp;
  if (c >= num_chunks) return;
  int* cur = cursors + warp * nbins;
  for (int b = lane; b < nbins; b += 32) cur[b] = bin_base[b] + partial[int64_t(b) * num_chunks + c];
  __syncwarp();
  const int64_t begin = int64_t(c) * chunk;
  const int64_t end = min(begin + chunk, n);
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t i = base + lane;
    const bool valid = i < end;
    K key = valid ? keys[i] : K(0);
    const int d = valid ? digit_of(key, shift, bits, flip_sign) : -1 - lane;  // invalid lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, d);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int pos = 0;
    if (valid) pos = cur[d] + rank;
    __syncwarp();
    if (valid && rank == 0) cur[d] += __popc(peers);
    __syncwarp();
    if (valid) {
      keys_out[pos] = key;
      vals_out[pos] = vals_in != nullptr ? vals_in[i] : static_cast<V>(i);
    }
  }
}

}  // namespace

int sort_warp_chunk(int64_t n) { return warp_chunk(n); }

cudaError_t sort_pass(DType key_type, const void* keys, const void* vals_in, int64_t n, int shift, int bits,
                      bool flip_sign, int chunk, int num_chunks, int* partial, int* totals, void* keys_out,
                      void* vals_out, int* tpe, int* bins, int* padded_bins, int num_real_bins, int block,
                      cudaStream_t stream) {
  const int nbins = 1 << bits;
  const int grid = ceil_div(num_chunks, kSortWarps);
  const size_t hist_smem = size_t(kSortWarps) * nbins * sizeof(int);
  const size_t place_smem = size_t(nbins + 8 + kSortWarps * nbins) * sizeof(int);
  MB_SWITCH_INT(key_type, K, {
    sort_hist_kernel<K><<<grid, kSortThreads, hist_smem, stream>>>(static_cast<const K*>(keys), n, shift, bits,
                                                                    flip_sign, chunk, num_chunks, partial);
    sort_scan_kernel<<<nbins, 256, 0, stream>>>(partial, num_chunks, totals);
    // Values carry the key dtype (the reference returns the permutation in it).
    sort_place_kernel<K, K><<<grid, kSortThreads, place_smem, stream>>>(
        static_cast<const K*>(keys), static_cast<const K*>(vals_in), n, shift, bits, flip_sign, chunk, num_chunks,
        partial, totals, static_cast<K*>(keys_out), static_cast<K*>(vals_out), tpe, bins, padded_bins,
        num_real_bins, block);
  })
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// histogram
// ---------------------------------------------------------------------------
namespace {

constexpr int kHistSmemBins = 8192;

template <typename K>
__global__ void __launch_bounds__(256) histogram_kernel(const K* __restrict__ x, int64_t n, int num_bins,
                                                        int* __restrict__ out, bool use_smem) {
  extern __shared__ int hist[];
  const K* row = x + int64_t(blockIdx.y) * n;
  int* out_row = out + int64_t(blockIdx.y) * num_bins;
  if (use_smem) {
    for (int b = threadIdx.x; b < num_bins; b += blockDim.x) hist[b] = 0;
    __syncthreads();
  }
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t v = static_cast<int64_t>(row[i]);
    if (v >= 0 && v < num_bins) atomicAdd(use_smem ? &hist[v] : &out_row[v], 1);
  }
  if (use_smem) {
    __syncthreads();
    for (int b = threadIdx.x; b < num_bins; b += blockDim.x)
      if (hist[b]) atomicAdd(&out_row[b], hist[b]);
  }
}

}  // namespace

cudaError_t histogram(DType type, const void* x, int64_t batch, int64_t n, int num_bins, int* out, int sms,
                      cudaStream_t stream) {
  const bool use_smem = num_bins <= kHistSmemBins;
  const int blocks = max(1, min(ceil_div(n, 256 * 8), 4 * sms));
  dim3 grid(blocks, static_cast<unsigned>(batch));
  MB_SWITCH_INT(type, K, {
    histogram_kernel<K><<<grid, 256, use_smem ? num_bins * sizeof(int) : 0, stream>>>(
        static_cast<const K*>(x), n, num_bins, out, use_smem);
  })
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// row-wise prefix sums
// ---------------------------------------------------------------------------
namespace {

template <typename K>
__global__ void __launch_bounds__(256) cumsum_kernel(const K* __restrict__ x, K* __restrict__ out, int64_t cols,
                                                     bool exclusive) {
  constexpr int kItems = 4;
  __shared__ long long warp_sums[8];
  __shared__ long long carry_s;
  const K* row = x + int64_t(blockIdx.x) * cols;
  K* orow = out + int64_t(blockIdx.x) * cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < cols; base += 256 * kItems) {
    const int64_t first = base + int64_t(threadIdx.x) * kItems;
    long long v[kItems];
    long long sum = 0;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      v[j] = (first + j < cols) ? static_cast<long long>(row[first + j]) : 0;
      sum += v[j];
    }
    long long incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      long long t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    long long off = carry_s + incl - sum;
    for (int w = 0; w < warp; ++w) off += warp_sums[w];
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      if (first + j < cols) orow[first + j] = static_cast<K>(exclusive ? off : off + v[j]);
      off += v[j];
    }
    __syncthreads();
    if (threadIdx.x == 255) carry_s = off;
    __syncthreads();
  }
}

}  // namespace

cudaError_t cumsum(DType type, const void* x, void* out, int64_t rows, int64_t cols, bool exclusive,
                   cudaStream_t stream) {
  MB_SWITCH_INT(type, K, {
    cumsum_kernel<K><<<static_cast<unsigned>(rows), 256, 0, stream>>>(static_cast<const K*>(x),
                                                                      static_cast<K*>(out), cols, exclusive);
  })
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// topology
// ---------------------------------------------------------------------------
namespace {

__global__ void topology_kernel(const int* __restrict__ padded_bins, int num_bins, int block_size, int rows,
                                int cols, int16_t* __restrict__ out) {
  const int64_t total = int64_t(rows) * cols;
  for (int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / cols);
    const int col = static_cast<int>(idx - int64_t(row) * cols);
    // Expert of this row-block: first bin whose padded end (in rows) exceeds row*block.
    const int e = upper_bound_i32(padded_bins, num_bins, row * block_size);
    out[idx] = e < num_bins ? static_cast<int16_t>(e * cols + col) : int16_t(0);
  }
}

}  // namespace

cudaError_t topology(const int* padded_bins, int num_bins, int block_size, int rows, int cols, int16_t* out,
                     int sms, cudaStream_t stream) {
  const int blocks = max(1, min(ceil_div(int64_t(rows) * cols, 256), 8 * sms));
  topology_kernel<<<blocks, 256, 0, stream>>>(padded_bins, num_bins, block_size, rows, cols, out);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// replicate
// ---------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void replicate_fwd_kernel(const T* __restrict__ x, const int* __restrict__ bins, int num_bins,
                                     int64_t num_outputs, T* __restrict__ out) {
  const T* xrow = x + int64_t(blockIdx.y) * num_bins;
  T* orow = out + int64_t(blockIdx.y) * num_outputs;
  for (int64_t j = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; j < num_outputs;
       j += int64_t(gridDim.x) * blockDim.x) {
    const int b = upper_bound_i32(bins, num_bins, static_cast<int>(j));
    orow[j] = b < num_bins ? xrow[b] : T(0);
  }
}

template <typename T>
__global__ void replicate_bwd_kernel(const T* __restrict__ grad, const int* __restrict__ bins, int num_bins,
                                     int64_t num_inputs, T* __restrict__ out) {
  // One warp per (batch row, bin): fp32 segmented sum.
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= num_bins) return;
  const T* grow = grad + int64_t(blockIdx.y) * num_inputs;
  const int begin = warp == 0 ? 0 : bins[warp - 1];
  const int end = bins[warp];
  float acc = 0.f;
  for (int j = begin + lane; j < end; j += 32) acc += to_float(grow[j]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) out[int64_t(blockIdx.y) * num_bins + warp] = from_float<T>(acc);
}

}  // namespace

cudaError_t replicate_fwd(int elem_size, const void* x, const int* bins, int num_bins, int64_t batch,
                          int64_t num_outputs, void* out, int sms, cudaStream_t stream) {
  dim3 grid(max(1, min(ceil_div(num_outputs, 256), 4 * sms)), static_cast<unsigned>(batch));
  switch (elem_size) {
    case 2:
      replicate_fwd_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(x), bins, num_bins,
                                                               num_outputs, static_cast<uint16_t*>(out));
      break;
    case 4:
      replicate_fwd_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(x), bins, num_bins,
                                                               num_outputs, static_cast<uint32_t*>(out));
      break;
    case 8:
      replicate_fwd_kernel<uint64_t><<<grid, 256, 0, stream>>>(static_cast<const uint64_t*>(x), bins, num_bins,
                                                               num_outputs, static_cast<uint64_t*>(out));
      break;
    default:
      return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t replicate_bwd(DType type, const void* grad, const int* bins, int num_bins, int64_t batch,
                          int64_t num_inputs, void* out, cudaStream_t stream) {
  dim3 grid(ceil_div(int64_t(num_bins) * 32, 256), static_cast<unsigned>(batch));
  MB_SWITCH_FLOAT(type, T, {
    replicate_bwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(grad), bins, num_bins, num_inputs,
                                                      static_cast<T*>(out));
  })
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free route plan (see route_plan_noalloc.h)
// ---------------------------------------------------------------------------
namespace {

// Scratch of one counting-sort pass at the stated maxima: per-chunk histograms
// [1024 bins][512 chunks] followed by the 1024 bin totals.
constexpr int kNoAllocMaxChunks = MB_NOALLOC_MAX_COPIES / 2048;
constexpr int kNoAllocPartialInts = MB_NOALLOC_MAX_EXPERTS * kNoAllocMaxChunks;
constexpr int kNoAllocScratchInts = kNoAllocPartialInts + MB_NOALLOC_MAX_EXPERTS;

static __device__ __align__(256) int g_noalloc_scratch[kNoAllocScratchInts];

// Device address of the scratch array per device.  The array's name is only a
// host-side handle; kernels need the address cudaGetSymbolAddress reports.
// (Filled on first use; two host threads that race here store the same value, and the atomic makes
// that exchange well defined.)
std::atomic<int*> g_noalloc_scratch_addr[64];

cudaError_t noalloc_scratch(int** out) {
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  int* addr = g_noalloc_scratch_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* ptr = nullptr;
    rc = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (rc != cudaSuccess) return rc;
    addr = static_cast<int*>(ptr);
    g_noalloc_scratch_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return cudaSuccess;
}

}  // namespace

}  // namespace mb

extern "C" cudaError_t mb_route_plan_noalloc(const int32_t* top_experts, int64_t n, int num_experts, int block,
                                             int32_t* indices, int32_t* bin_ids, int32_t* bins,
                                             int32_t* padded_bins, int32_t* tokens_per_expert,
                                             cudaStream_t stream) {
  using namespace mb;
  if (n < 0 || n > MB_NOALLOC_MAX_COPIES || num_experts < 1 || num_experts > MB_NOALLOC_MAX_EXPERTS || block < 1) {
    std::fprintf(stderr,
                 "mb_route_plan_noalloc: n=%lld experts=%d block=%d is outside the supported range "
                 "(n <= %d, 1 <= experts <= %d, block >= 1)\n",
                 static_cast<long long>(n), num_experts, block, MB_NOALLOC_MAX_COPIES, MB_NOALLOC_MAX_EXPERTS);
    return cudaErrorInvalidValue;
  }
  int* scratch = nullptr;
  cudaError_t rc = noalloc_scratch(&scratch);
  if (rc != cudaSuccess) return rc;
  int bits = 1;
  while ((1 << bits) < num_experts) ++bits;
  const int chunk = sort_warp_chunk(n);
  const int num_chunks = n > 0 ? ceil_div(n, chunk) : 1;
  if (int64_t(1 << bits) * num_chunks > kNoAllocPartialInts) return cudaErrorInvalidValue;
  int* partial = scratch;
  int* totals = scratch + kNoAllocPartialInts;
  if (n == 0) {
    // No copies: the counts and both prefix sums are all zero.
    rc = cudaMemsetAsync(tokens_per_expert, 0, sizeof(int) * num_experts, stream);
    if (rc == cudaSuccess) rc = cudaMemsetAsync(bins, 0, sizeof(int) * num_experts, stream);
    if (rc == cudaSuccess) rc = cudaMemsetAsync(padded_bins, 0, sizeof(int) * num_experts, stream);
    return rc;
  }
  // One stable pass over the expert-id bits.  Every scratch word that the scan and
  // placement kernels read is written by the histogram kernel of this same call, so
  // nothing needs clearing.
  return sort_pass(kI32, top_experts, nullptr, n, 0, bits, false, chunk, num_chunks, partial, totals, bin_ids,
                   indices, tokens_per_expert, bins, padded_bins, num_experts, block, stream);
}
