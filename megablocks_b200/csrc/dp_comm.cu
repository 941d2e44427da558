// Data-parallel gradient reduction over NVLink / NVSwitch peer memory (sm_100a).
//
// The reference leaves data parallelism to its outer trainer, which all-reduces the non-expert
// gradients with NCCL (exp/dmoe/dmoe_125m_8gpu.sh:145, `--DDP-impl local`).  Here the replicated
// gradients of every rank live in a symmetric heap that all ranks map, and ONE kernel per gradient
// bucket does the whole collective with plain peer loads and stores, launched from the backward
// hooks on a side stream so that it overlaps the rest of backward:
//
//   1. every rank releases a "bucket ready" flag in every peer and waits for all peers' flags;
//   2. rank r owns slice r of the bucket: it loads that slice from every rank (16-byte peer loads,
//      several in flight per thread), sums in fp32 in rank order, scales, and stores the result
//      into slice r of every rank (all-reduce) or only of itself (reduce-scatter, ZeRO-1).  Each
//      element is reduced by exactly one rank, so all ranks end up with bitwise identical values;
//   3. the last CTA to finish releases a "bucket done" flag in every peer and waits for all peers'
//      flags: when the kernel ends, every slice of this rank's bucket has been written by its
//      owner and no peer still reads this rank's gradients.
//
// Flags carry a sequence number (one per step), so nothing is ever reset.  Every wait is bounded;
// on expiry a code is recorded in the status word and the kernel returns.  A kernel that finds a
// recorded failure on entry does nothing.
#include "common.cuh"

namespace mb {

namespace {

constexpr uint64_t kDpWaitLimitNs = 2000000000ull;
constexpr int kDpThreads = 512;
constexpr int kDpUnroll = 4;

__device__ __forceinline__ uint64_t dp_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void dp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int dp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool dp_wait_flag(const int* flag, int target, int* status, int code) {
  if (dp_ld_acquire_sys(flag) >= target) return true;
  const uint64_t t0 = dp_timer_ns();
  uint32_t spins = 0;
  while (dp_ld_acquire_sys(flag) < target) {
    if ((++spins & 63u) == 0u) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (dp_timer_ns() - t0 > kDpWaitLimitNs) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
// Peer gradients are read once and are being rewritten by their owner's next step: bypass L1.
__device__ __forceinline__ uint4 dp_ld_peer(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ void dp_accumulate(const uint4& raw, float (&acc)[16 / sizeof(T)]) {
  const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < int(16 / sizeof(T)); ++i) acc[i] += to_float(v[i]);
}

template <typename T>
__global__ void __launch_bounds__(kDpThreads)
dp_allreduce_kernel(DpLayout L, int64_t start, int64_t count, int bucket, int seq, float scale, int scatter_only,
                    int* __restrict__ ticket, int* status) {
  constexpr int VEC = 16 / sizeof(T);
  const int W = L.world;
  if (L.seq_base != nullptr) seq += *L.seq_base;
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = *reinterpret_cast<volatile int*>(status) == 0;
  __syncthreads();
  if (!ok_s) return;
  // ---- 1. ready ---------------------------------------------------------------------
  if (blockIdx.x == 0 && threadIdx.x < W)
    dp_st_release_sys(reinterpret_cast<int*>(L.peer_base[threadIdx.x] + L.off_ready) + bucket * W + L.rank, seq);
  if (threadIdx.x < W) {
    const int* mine = reinterpret_cast<const int*>(L.peer_base[L.rank] + L.off_ready) + bucket * W + threadIdx.x;
    if (!dp_wait_flag(mine, seq, status, kDpErrReady)) ok_s = 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // ---- 2. reduce my slice, publish it ----------------------------------------------------
  // 16-byte vectors of the bucket are dealt to the ranks in contiguous runs; the last run may be short.
  const int64_t total_vecs = count / VEC;
  const int64_t per_rank = (total_vecs + W - 1) / W;
  const int64_t first = min(int64_t(L.rank) * per_rank, total_vecs);
  const int64_t vecs = min(per_rank, total_vecs - first);
  const int64_t begin = start + first * VEC;
  const int64_t stride = int64_t(gridDim.x) * kDpThreads;
  for (int64_t v0 = int64_t(blockIdx.x) * kDpThreads + threadIdx.x; v0 < vecs; v0 += stride * kDpUnroll) {
    float acc[kDpUnroll][VEC];
#pragma unroll
    for (int u = 0; u < kDpUnroll; ++u)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[u][i] = 0.f;
    for (int r = 0; r < W; ++r) {
      const T* src = reinterpret_cast<const T*>(L.peer_base[r] + L.off_grad) + begin;
      uint4 raw[kDpUnroll];
#pragma unroll
      for (int u = 0; u < kDpUnroll; ++u) {
        const int64_t v = v0 + u * stride;
        if (v < vecs) raw[u] = dp_ld_peer(src + v * VEC);
      }
#pragma unroll
      for (int u = 0; u < kDpUnroll; ++u)
        if (v0 + u * stride < vecs) dp_accumulate<T>(raw[u], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < kDpUnroll; ++u) {
      const int64_t v = v0 + u * stride;
      if (v >= vecs) continue;
      uint4 packed;
      T* out = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int i = 0; i < VEC; ++i) out[i] = from_float<T>(acc[u][i] * scale);
      if (scatter_only) {
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(L.peer_base[L.rank] + L.off_grad) + begin + v * VEC) = packed;
      } else {
        for (int r = 0; r < W; ++r)
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(L.peer_base[r] + L.off_grad) + begin + v * VEC) = packed;
      }
    }
  }
  // ---- 3. done ------------------------------------------------------------------------
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last_s = atomicAdd(ticket, 1) == int(gridDim.x) - 1;
    if (last_s) *ticket = 0;          // ready for the bucket's next launch
  }
  __syncthreads();
  if (!last_s) return;
  if (threadIdx.x < W) {
    __threadfence_system();           // the other CTAs' stores were fenced before their tickets
    dp_st_release_sys(reinterpret_cast<int*>(L.peer_base[threadIdx.x] + L.off_done) + bucket * W + L.rank, seq);
    const int* mine = reinterpret_cast<const int*>(L.peer_base[L.rank] + L.off_done) + bucket * W + threadIdx.x;
    dp_wait_flag(mine, seq, status, kDpErrDone);
  }
}

}  // namespace

cudaError_t dp_allreduce(DType type, const DpLayout& layout, int64_t start, int64_t count, int bucket, int seq,
                         float scale, bool scatter_only, int* ticket, int* status, int ctas, cudaStream_t stream) {
  const int elem = type == kF32 ? 4 : 2;
  const int vec = 16 / elem;
  if (layout.world < 1 || layout.world > kDpThreads || count < 0 || count % vec != 0 || (start * elem) % 16 != 0 ||
      (layout.off_grad % 16) != 0)
    return cudaErrorInvalidValue;
  if (count == 0) return cudaSuccess;
  const int grid = max(1, min(ctas, ceil_div(ceil_div(count / vec, layout.world), kDpThreads)));
  MB_SWITCH_FLOAT(type, T, {
    dp_allreduce_kernel<T><<<grid, kDpThreads, 0, stream>>>(layout, start, count, bucket, seq, scale,
                                                            scatter_only ? 1 : 0, ticket, status);
  })
  return cudaGetLastError();
}

}  // namespace mb
