// Expert-parallel exchange kernels over NVLink / NVSwitch peer memory (sm_100a).
//
// The reference moves tokens between expert-parallel ranks with three NCCL
// all-to-alls per layer and direction plus a device-to-host copy of the counts
// (megablocks/layers/moe.py:237-423 of the reference).  Here every rank maps every
// peer's workspace (one symmetric heap per group) and the kernels below store rows
// straight into the owner's expert-ordered buffer, publish per-expert release flags,
// and never involve the host:
//
//   ep_exchange_counts  every rank writes its per-expert copy counts into every
//                       peer's count matrix, then waits for all peers (bounded) and
//                       derives the receive-side prefix sums;
//   ep_push_rows        token order -> owner's expert order.  Row i of my sorted
//                       copies (expert e) lands at
//                         owner_base(e) + sum_{s < me} count[s][e] + (i - start(e))
//                       in the owner's buffer.  When the last row of (me, e) has been
//                       stored the owner's flag[me][e_local] is released, so the
//                       owner's GEMM can start on an expert the moment all sources have
//                       delivered it (the GEMM producer warp polls those flags);
//   ep_return_rows      owner's expert order -> the source's sorted order, with one
//                       release flag per (owner, source);
//   ep_wait_flags       a one-CTA bounded wait used in front of kernels that read a
//                       whole returned buffer.
//
// Only plain peer loads/stores and system-scope release/acquire are used.  Every
// wait is bounded by a timeout; on expiry a code is written to the status word and
// the kernel returns.
#include "common.cuh"

namespace mb {

namespace {

constexpr uint64_t kEpWaitLimitNs = 2000000000ull;
constexpr int kPushWarps = 8;

__device__ __forceinline__ uint64_t ep_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *flag >= target, at most kEpWaitLimitNs.  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const int* flag, int target, int* status, int code) {
  if (ld_acquire_sys(flag) >= target) return true;
  const uint64_t t0 = ep_timer_ns();
  uint32_t spins = 0;
  while (ld_acquire_sys(flag) < target) {
    if ((++spins & 63u) == 0u) {
      // A failure already recorded on this device ends every later wait at once.
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (ep_timer_ns() - t0 > kEpWaitLimitNs) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

template <typename T>
__device__ __forceinline__ T* peer_ptr(const uint64_t* peer_base, int rank, int64_t byte_offset) {
  return reinterpret_cast<T*>(peer_base[rank] + byte_offset);
}

// ---------------------------------------------------------------------------
// counts
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
exchange_counts_kernel(const int* __restrict__ tpe, EpLayout L, int seq, int expert_capacity,
                       int* __restrict__ counts_out, int* __restrict__ kept_out, int* __restrict__ recv_bins,
                       int* __restrict__ scratch_zero, int scratch_ints, int* status) {
  if (L.seq_base != nullptr) seq += *L.seq_base;
  const int parity = seq & 1;
  const int64_t counts_off = L.off_counts + int64_t(parity) * L.world * L.num_experts * 4;
  // (a) my counts -> row `me` of every peer's matrix.
  for (int e = threadIdx.x; e < L.num_experts; e += blockDim.x) {
    const int v = tpe[e];
    for (int r = 0; r < L.world; ++r)
      peer_ptr<int>(L.peer_base, r, counts_off)[L.rank * L.num_experts + e] = v;
  }
  for (int i = threadIdx.x; i < scratch_ints; i += blockDim.x) scratch_zero[i] = 0;
  __threadfence_system();
  __syncthreads();
  // (b) release one flag per peer, (c) wait for every peer's flag.
  if (threadIdx.x < L.world)
    st_release_sys(peer_ptr<int>(L.peer_base, threadIdx.x, L.off_count_flags) + L.rank, seq);
  __shared__ int ok_s, dead_s;
  if (threadIdx.x == 0) {
    ok_s = 1;
    dead_s = *reinterpret_cast<volatile int*>(status) != 0;   // an earlier failure on this device
  }
  __syncthreads();
  if (threadIdx.x < L.world) {
    const int* mine = peer_ptr<int>(L.peer_base, L.rank, L.off_count_flags) + threadIdx.x;
    if (!wait_flag(mine, seq, status, kEpErrCounts)) ok_s = 0;
  }
  __syncthreads();
  if (!ok_s || dead_s) {
    // Fail closed: with an all-zero count matrix every kernel that follows on this stream
    // (push, expert GEMMs, return) finds nothing to move and stores nothing anywhere.
    for (int i = threadIdx.x; i < L.world * L.num_experts; i += blockDim.x) counts_out[i] = kept_out[i] = 0;
    for (int j = threadIdx.x; j < L.experts_per_rank; j += blockDim.x) recv_bins[j] = 0;
    return;
  }
  // (d) local copy of the matrix and receive-side prefix sums.  A count outside [0, copy_bound]
  // cannot come from a healthy peer; it is treated like an overflow.
  const int* counts = peer_ptr<int>(L.peer_base, L.rank, counts_off);
  __shared__ int bad_s;
  if (threadIdx.x == 0) bad_s = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < L.world * L.num_experts; i += blockDim.x) {
    int v = ld_acquire_sys(counts + i);
    if (v < 0 || v > L.capacity_rows) { v = 0; bad_s = 1; }
    counts_out[i] = v;
  }
  __syncthreads();
  // Rows that survive a per-expert capacity: of everything routed to expert e, taken source by
  // source in rank order, only the first `expert_capacity` rows are kept (0 = no limit), which is
  // the rule of the reference's binned gather after its second sort.
  for (int e = threadIdx.x; e < L.num_experts; e += blockDim.x) {
    int room = expert_capacity > 0 ? expert_capacity : 0x7fffffff;
    for (int s = 0; s < L.world; ++s) {
      const int keep = min(counts_out[s * L.num_experts + e], room);
      kept_out[s * L.num_experts + e] = keep;
      room -= keep;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int j = 0; j < L.experts_per_rank; ++j) {
      const int e = L.rank * L.experts_per_rank + j;
      for (int s = 0; s < L.world; ++s) acc += kept_out[s * L.num_experts + e];
      // More rows than the buffer holds: the senders skip them (see push_rows_kernel), the
      // receiver's groups end at the capacity, and the status word reports the overflow.
      recv_bins[j] = min(acc, L.capacity_rows);
    }
    if (acc > L.capacity_rows || bad_s) atomicCAS(status, 0, kEpErrOverflow);
  }
}

// ---------------------------------------------------------------------------
// push: my sorted copies -> owners
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kPushWarps * 32)
push_rows_kernel(const T* __restrict__ x, const int* __restrict__ indices, const T* __restrict__ weights,
                 const int* __restrict__ bins, const int* __restrict__ counts, EpLayout L,
                 const uint64_t* __restrict__ data_base, int64_t off_recv, int64_t off_flags, int64_t off_free,
                 int seq, int top_k, int n, int cols, int* __restrict__ done, int* status,
                 T* __restrict__ dropped_rows) {
  extern __shared__ int smem[];
  if (L.seq_base != nullptr) seq += *L.seq_base;
  int* dst_start = smem;                    // [E] first row of (me, e) in the owner's buffer
  int* src_start = smem + L.num_experts;    // [E] first sorted position of e here
  const int E = L.num_experts, W = L.world, epr = L.experts_per_rank;
  // A recorded failure (a peer that never answered, an overflow) makes the exchange inert:
  // nothing is stored into any peer and no flag is released.
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / epr) * epr;
    int acc = 0;
    for (int e2 = first; e2 < e; ++e2)
      for (int s = 0; s < W; ++s) acc += counts[s * E + e2];
    for (int s = 0; s < L.rank; ++s) acc += counts[s * E + e];
    dst_start[e] = acc;
    src_start[e] = e ? bins[e - 1] : 0;
    // An expert I send nothing to still needs its flag so the owner does not wait for me.
    if (blockIdx.x == 0 && bins[e] - src_start[e] == 0)
      st_release_sys(peer_ptr<int>(L.peer_base, e / epr, off_flags) + L.rank * epr + (e - first), seq);
  }
  // The owners' receive buffer of the previous use must have been read completely
  // (each owner publishes the last sequence number it is done with).
  __shared__ int free_ok;
  if (threadIdx.x == 0) free_ok = 1;
  __syncthreads();
  if (off_free >= 0 && threadIdx.x < W) {
    if (!wait_flag(peer_ptr<int>(L.peer_base, threadIdx.x, off_free), seq - 1, status, kEpErrBufferBusy))
      free_ok = 0;
  }
  __syncthreads();
  if (!free_ok) return;
  const int lane = threadIdx.x & 31;
  constexpr int VEC = 16 / sizeof(T);
  // Every CTA owns one contiguous range of sorted positions: it touches few experts, and
  // one system-scope fence per CTA (instead of one per row) orders all its stores before
  // the completion counters and flags.
  const int per_cta = (n + gridDim.x - 1) / gridDim.x;
  const int begin = min(n, blockIdx.x * per_cta), end = min(n, begin + per_cta);
  for (int i = begin + (threadIdx.x >> 5); i < end; i += kPushWarps) {
    const int e = upper_bound_i32(bins, E, i);
    const int owner = e / epr;
    const int copy = __ldg(indices + i);
    const T* src = x + int64_t(copy / top_k) * cols;
    if (e >= E) continue;
    const int within = i - src_start[e];
    if (within >= counts[L.rank * E + e]) {
      // Beyond the expert's capacity: the copy is dropped.  Nobody will return a row for it, so its
      // slot in this rank's return buffer is cleared here.
      if (dropped_rows != nullptr)
        for (int c0 = lane * VEC; c0 < cols; c0 += 32 * VEC)
          *reinterpret_cast<uint4*>(dropped_rows + int64_t(i) * cols + c0) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int dst_row = dst_start[e] + within;
    if (dst_row < 0 || dst_row >= L.capacity_rows) continue;   // never store outside the owner's buffer
    T* dst = peer_ptr<T>(data_base, owner, off_recv) + int64_t(dst_row) * cols;
    const float scale = weights != nullptr ? to_float(weights[copy]) : 1.f;
    // Four 16-byte loads in flight per lane before the first (remote) store.
    for (int c0 = lane * VEC; c0 < cols; c0 += 4 * 32 * VEC) {
      uint4 raw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32 * VEC;
        if (c < cols) raw[j] = *reinterpret_cast<const uint4*>(src + c);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32 * VEC;
        if (c < cols) {
          if (weights != nullptr) {
            T* v = reinterpret_cast<T*>(&raw[j]);
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[k] = from_float<T>(to_float(v[k]) * scale);
          }
          *reinterpret_cast<uint4*>(dst + c) = raw[j];
        }
      }
    }
  }
  __syncthreads();
  if (end > begin && threadIdx.x == 0) {
    __threadfence_system();
    const int e_first = upper_bound_i32(bins, E, begin), e_last = upper_bound_i32(bins, E, end - 1);
    for (int e = e_first; e <= e_last; ++e) {
      const int lo = max(begin, src_start[e]), hi = min(end, bins[e]);
      if (hi <= lo) continue;
      const int total = bins[e] - src_start[e];
      if (atomicAdd(done + e, hi - lo) + (hi - lo) == total) {
        __threadfence_system();   // other CTAs' rows of this expert were fenced before their adds
        const int owner = e / epr;
        st_release_sys(peer_ptr<int>(L.peer_base, owner, off_flags) + L.rank * epr + (e - owner * epr), seq);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// return: my expert-ordered rows -> the sources' sorted order
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kPushWarps * 32)
return_rows_kernel(const T* __restrict__ y, const int* __restrict__ counts, const int* __restrict__ raw_counts,
                   EpLayout L,
                   const uint64_t* __restrict__ data_base, int64_t off_ret, int64_t off_flags, int seq, int cols,
                   int rows_bound, int ret_rows, int* __restrict__ done, const int* status) {
  extern __shared__ int smem[];
  if (L.seq_base != nullptr) seq += *L.seq_base;
  const int E = L.num_experts, W = L.world, epr = L.experts_per_rank;
  if (*reinterpret_cast<const volatile int*>(status) != 0) return;   // inert after a recorded failure
  int* seg_end = smem;                 // [epr * W] inclusive end row of segment (j, s) here
  int* remote_start = smem + epr * W;  // [epr * W] first sorted position of (s, e_j) at source s
  int* per_source = smem + 2 * epr * W;  // [W] rows I return to source s
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int j = 0; j < epr; ++j)
      for (int s = 0; s < W; ++s) {
        acc += counts[s * E + L.rank * epr + j];
        seg_end[j * W + s] = acc;
      }
  }
  for (int idx = threadIdx.x; idx < epr * W; idx += blockDim.x) {
    const int j = idx / W, s = idx - j * W;
    const int e = L.rank * epr + j;
    int acc = 0;
    for (int e2 = 0; e2 < e; ++e2) acc += raw_counts[s * E + e2];   // the source's order holds dropped copies too
    remote_start[idx] = acc;
  }
  for (int s = threadIdx.x; s < W; s += blockDim.x) {
    int acc = 0;
    for (int j = 0; j < epr; ++j) acc += counts[s * E + L.rank * epr + j];
    per_source[s] = acc;
    if (blockIdx.x == 0 && acc == 0)
      st_release_sys(peer_ptr<int>(L.peer_base, s, off_flags) + L.rank, seq);
  }
  __syncthreads();
  const int total = min(seg_end[epr * W - 1], rows_bound);   // never read past y
  const int lane = threadIdx.x & 31;
  constexpr int VEC = 16 / sizeof(T);
  // Contiguous row range per CTA; one system-scope fence per CTA (see push_rows_kernel).
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int begin = min(total, blockIdx.x * per_cta), end = min(total, begin + per_cta);
  for (int row = begin + (threadIdx.x >> 5); row < end; row += kPushWarps) {
    // Segment of this row: first (j, s) whose end exceeds it.
    int lo = 0, hi = epr * W;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (seg_end[mid] <= row) lo = mid + 1; else hi = mid;
    }
    const int s = lo % W;
    const int seg_begin = lo ? seg_end[lo - 1] : 0;
    const int remote_row = remote_start[lo] + (row - seg_begin);
    if (lo >= epr * W || remote_row < 0 || remote_row >= ret_rows) continue;   // outside the source's buffer
    const T* src = y + int64_t(row) * cols;
    T* dst = peer_ptr<T>(data_base, s, off_ret) + int64_t(remote_row) * cols;
    for (int c0 = lane * VEC; c0 < cols; c0 += 4 * 32 * VEC) {
      uint4 raw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32 * VEC;
        if (c < cols) raw[j] = *reinterpret_cast<const uint4*>(src + c);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32 * VEC;
        if (c < cols) *reinterpret_cast<uint4*>(dst + c) = raw[j];
      }
    }
  }
  __syncthreads();
  if (end > begin && threadIdx.x == 0) {
    __threadfence_system();
    int seg = 0;
    {
      int lo = 0, hi = epr * W;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (seg_end[mid] <= begin) lo = mid + 1; else hi = mid;
      }
      seg = lo;
    }
    for (; seg < epr * W; ++seg) {
      const int seg_begin = seg ? seg_end[seg - 1] : 0;
      if (seg_begin >= end) break;
      const int lo = max(begin, seg_begin), hi = min(end, seg_end[seg]);
      if (hi <= lo) continue;
      const int s = seg % W;
      if (atomicAdd(done + s, hi - lo) + (hi - lo) == per_source[s]) {
        __threadfence_system();
        st_release_sys(peer_ptr<int>(L.peer_base, s, off_flags) + L.rank, seq);
      }
    }
  }
}

__global__ void wait_flags_kernel(const int* flags, int count, int seq, const int* seq_base, int* status, int code) {
  if (seq_base != nullptr) seq += *seq_base;
  if (threadIdx.x < count) wait_flag(flags + threadIdx.x, seq, status, code);
}

__global__ void set_flag_kernel(int* flag, int value, const int* seq_base) {
  st_release_sys(flag, value + (seq_base != nullptr ? *seq_base : 0));
}

}  // namespace

cudaError_t ep_exchange_counts(const int* tpe, const EpLayout& layout, int seq, int expert_capacity, int* counts_out,
                               int* kept_out, int* recv_bins, int* scratch_zero, int scratch_ints, int* status,
                               cudaStream_t stream) {
  if (layout.world > 1024) return cudaErrorInvalidValue;
  exchange_counts_kernel<<<1, 1024, 0, stream>>>(tpe, layout, seq, expert_capacity, counts_out, kept_out, recv_bins,
                                                scratch_zero, scratch_ints, status);
  return cudaGetLastError();
}

cudaError_t ep_push_rows(DType type, const void* x, const int* indices, const void* weights, const int* bins,
                         const int* counts, const EpLayout& layout, const uint64_t* data_base, int64_t off_recv,
                         int64_t off_flags, int64_t off_free, int seq, int top_k, int n, int cols, int* done,
                         int* status, void* dropped_rows, int sms, cudaStream_t stream) {
  const int elem = type == kF32 ? 4 : 2;
  if ((int64_t(cols) * elem) % 16 != 0) return cudaErrorInvalidValue;
  const int grid = max(1, min(ceil_div(max(n, 1), kPushWarps), sms * 4));
  const size_t smem = size_t(2) * layout.num_experts * sizeof(int);
  MB_SWITCH_FLOAT(type, T, {
    push_rows_kernel<T><<<grid, kPushWarps * 32, smem, stream>>>(
        static_cast<const T*>(x), indices, static_cast<const T*>(weights), bins, counts, layout, data_base, off_recv,
        off_flags, off_free, seq, top_k, n, cols, done, status, static_cast<T*>(dropped_rows));
  })
  return cudaGetLastError();
}

cudaError_t ep_return_rows(DType type, const void* y, const int* counts, const int* raw_counts,
                           const EpLayout& layout,
                           const uint64_t* data_base, int64_t off_ret, int64_t off_flags, int seq, int cols,
                           int rows_bound, int ret_rows, int* done, const int* status, int sms,
                           cudaStream_t stream) {
  const int elem = type == kF32 ? 4 : 2;
  if ((int64_t(cols) * elem) % 16 != 0) return cudaErrorInvalidValue;
  const int segs = layout.experts_per_rank * layout.world;
  const size_t smem = size_t(2 * segs + layout.world) * sizeof(int);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const int grid = max(1, min(ceil_div(max(rows_bound, 1), kPushWarps), sms * 4));
  MB_SWITCH_FLOAT(type, T, {
    return_rows_kernel<T><<<grid, kPushWarps * 32, smem, stream>>>(static_cast<const T*>(y), counts, raw_counts, layout,
                                                                  data_base, off_ret, off_flags, seq, cols, rows_bound,
                                                                  ret_rows, done, status);
  })
  return cudaGetLastError();
}

cudaError_t ep_wait_flags(const int* flags, int count, int seq, const int* seq_base, int* status, int code,
                          cudaStream_t stream) {
  if (count > 1024) return cudaErrorInvalidValue;
  wait_flags_kernel<<<1, 1024, 0, stream>>>(flags, count, seq, seq_base, status, code);
  return cudaGetLastError();
}

cudaError_t ep_set_flag(int* flag, int value, const int* seq_base, cudaStream_t stream) {
  set_flag_kernel<<<1, 1, 0, stream>>>(flag, value, seq_base);
  return cudaGetLastError();
}

}  // namespace mb
