// Row-wise fused kernels for the transformer around the MoE layers (sm_100a):
// softmax cross-entropy (forward and in-place backward, no fp32 copy of the logits)
// and LayerNorm (forward; backward with the weight / bias gradients reduced through
// shared memory and one small second pass).  The reference has no model code; these
// serve this library's own training model (models/transformer.py), where the eager
// PyTorch versions cost more HBM traffic than the whole MoE stack.
#include <cstdlib>

#include "common.cuh"

namespace mb {

namespace {

constexpr int kCeThreads = 512;

template <typename T, int N>
struct alignas(16) Pack {
  T v[N];
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// lse[t] = log sum_j exp(x[t, j]);  loss[t] = lse[t] - x[t, target[t]].
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ targets, int64_t vocab,
                         float* __restrict__ lse_out, float* __restrict__ loss_out) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
  const T* row = logits + int64_t(blockIdx.x) * vocab;
  float m = -INFINITY, s = 0.f;
  const bool vec_ok = (vocab % VEC == 0) && (reinterpret_cast<uintptr_t>(row) % 16 == 0);
  auto add = [&](float x) {
    if (x > m) { s = s * __expf(m - x) + 1.f; m = x; } else { s += __expf(x - m); }
  };
  if (vec_ok) {
    for (int64_t i = int64_t(threadIdx.x) * VEC; i < vocab; i += kCeThreads * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(row + i);
      // One running-maximum update per pack (the exponential unit is the scarce resource here:
      // VEC + 1 exponentials per VEC elements instead of up to 2 * VEC).
      float v[VEC], pm = -INFINITY;
#pragma unroll
      for (int k = 0; k < VEC; ++k) { v[k] = to_float(p.v[k]); pm = fmaxf(pm, v[k]); }
      if (pm > m) { s *= __expf(m - pm); m = pm; }
      if (m != -INFINITY) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) s += __expf(v[k] - m);
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += kCeThreads) add(to_float(row[i]));
  }
  // Combine (m, s) pairs: warp, then block.
  const float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = wm; red_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x < 32) {
    float mm = threadIdx.x < kCeThreads / 32 ? red_m[threadIdx.x] : -INFINITY;
    float ss = threadIdx.x < kCeThreads / 32 ? red_s[threadIdx.x] : 0.f;
    const float bm = warp_max(mm);
    ss = warp_sum(mm == -INFINITY ? 0.f : ss * __expf(mm - bm));
    if (threadIdx.x == 0) {
      const float lse = bm + __logf(ss);
      lse_out[blockIdx.x] = lse;
      const int64_t tgt = targets[blockIdx.x];
      loss_out[blockIdx.x] = (tgt >= 0 && tgt < vocab) ? lse - to_float(row[tgt]) : 0.f;
    }
  }
}

// grad[t, j] = (exp(x[t, j] - lse[t]) - [j == target[t]]) * scale[0], written over x.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ targets, const float* __restrict__ lse,
                         const float* __restrict__ scale_ptr, float scale_mul, int64_t vocab) {
  constexpr int VEC = 16 / sizeof(T);
  T* row = logits + int64_t(blockIdx.x) * vocab;
  const float l = lse[blockIdx.x];
  const float scale = (scale_ptr != nullptr ? *scale_ptr : 1.f) * scale_mul;
  const int64_t tgt = targets[blockIdx.x];
  const bool valid = tgt >= 0 && tgt < vocab;
  const bool vec_ok = (vocab % VEC == 0) && (reinterpret_cast<uintptr_t>(row) % 16 == 0);
  if (vec_ok) {
    for (int64_t i = int64_t(threadIdx.x) * VEC; i < vocab; i += kCeThreads * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(row + i);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float g = valid ? __expf(to_float(p.v[k]) - l) : 0.f;
        if (i + k == tgt) g -= 1.f;
        p.v[k] = from_float<T>(g * scale);
      }
      *reinterpret_cast<Pack<T, VEC>*>(row + i) = p;
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += kCeThreads) {
      float g = valid ? __expf(to_float(row[i]) - l) : 0.f;
      if (i == tgt) g -= 1.f;
      row[i] = from_float<T>(g * scale);
    }
  }
}

// Loss and gradient in one launch: the row's log-sum-exp as in the forward kernel, then
// (exp(x - lse) - [j == target]) * scale written over the row.  The second pass reads the row a few
// microseconds after the first, from L2 (a row is 100 KB, a few hundred CTAs are in flight), so the
// logits cross the HBM bus once in each direction instead of twice in and once out.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_fused_kernel(T* __restrict__ logits, const int64_t* __restrict__ targets, int64_t vocab, float scale,
                           float* __restrict__ loss_out) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float red_m[kCeThreads / 32], red_s[kCeThreads / 32];
  __shared__ float lse_s;
  T* row = logits + int64_t(blockIdx.x) * vocab;
  const int64_t tgt = targets[blockIdx.x];
  const bool valid = tgt >= 0 && tgt < vocab;
  float m = -INFINITY, s = 0.f;
  const bool vec_ok = (vocab % VEC == 0) && (reinterpret_cast<uintptr_t>(row) % 16 == 0);
  if (vec_ok) {
    for (int64_t i = int64_t(threadIdx.x) * VEC; i < vocab; i += kCeThreads * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(row + i);
      float v[VEC], pm = -INFINITY;
#pragma unroll
      for (int k = 0; k < VEC; ++k) { v[k] = to_float(p.v[k]); pm = fmaxf(pm, v[k]); }
      if (pm > m) { s *= __expf(m - pm); m = pm; }
      if (m != -INFINITY) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) s += __expf(v[k] - m);
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += kCeThreads) {
      const float x = to_float(row[i]);
      if (x > m) { s = s * __expf(m - x) + 1.f; m = x; } else { s += __expf(x - m); }
    }
  }
  const float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = wm; red_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x < 32) {
    float mm = threadIdx.x < kCeThreads / 32 ? red_m[threadIdx.x] : -INFINITY;
    float ss = threadIdx.x < kCeThreads / 32 ? red_s[threadIdx.x] : 0.f;
    const float bm = warp_max(mm);
    ss = warp_sum(mm == -INFINITY ? 0.f : ss * __expf(mm - bm));
    if (threadIdx.x == 0) {
      const float lse = bm + __logf(ss);
      lse_s = lse;
      loss_out[blockIdx.x] = valid ? lse - to_float(row[tgt]) : 0.f;    // read before the row is overwritten
    }
  }
  __syncthreads();
  const float l = lse_s;
  if (vec_ok) {
    for (int64_t i = int64_t(threadIdx.x) * VEC; i < vocab; i += kCeThreads * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(row + i);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float g = valid ? __expf(to_float(p.v[k]) - l) : 0.f;
        if (i + k == tgt) g -= 1.f;
        p.v[k] = from_float<T>(g * scale);
      }
      *reinterpret_cast<Pack<T, VEC>*>(row + i) = p;
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += kCeThreads) {
      float g = valid ? __expf(to_float(row[i]) - l) : 0.f;
      if (i == tgt) g -= 1.f;
      row[i] = from_float<T>(g * scale);
    }
  }
}

// ---------------------------------------------------------------------------
// LayerNorm: one warp per row, rows strided over a persistent grid.
// ---------------------------------------------------------------------------
constexpr int kLnWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, int64_t rows,
                     int cols, float eps, T* __restrict__ y, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int rms) {
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + (threadIdx.x >> 5); r < rows; r += stride) {
    const T* xr = x + r * cols;
    float s = 0.f, ss = 0.f;
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) { const float v = to_float(p.v[k]); s += v; ss += v * v; }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    // RMS norm (`rms`): no centring and no bias; the stored mean is 0 so the backward needs no second form.
    const float mean = rms ? 0.f : s / cols;
    const float rstd = rsqrtf(fmaxf(ss / cols - mean * mean, 0.f) + eps);
    if (lane == 0) { mean_out[r] = mean; rstd_out[r] = rstd; }
    T* yr = y + r * cols;
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
      Pack<T, VEC> g = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
      Pack<T, VEC> b;
      if (beta != nullptr) b = *reinterpret_cast<const Pack<T, VEC>*>(beta + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k)
        p.v[k] = from_float<T>((to_float(p.v[k]) - mean) * rstd * to_float(g.v[k]) +
                               (beta != nullptr ? to_float(b.v[k]) : 0.f));
      *reinterpret_cast<Pack<T, VEC>*>(yr + c) = p;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                     const float* __restrict__ mean, const float* __restrict__ rstd, int64_t rows, int cols,
                     T* __restrict__ dx, float* __restrict__ partial, int rms) {
  constexpr int VEC = 16 / sizeof(T);
  extern __shared__ float acc[];          // [2][cols]: dgamma, dbeta of this CTA
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) acc[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + (threadIdx.x >> 5); r < rows; r += stride) {
    const T* xr = x + r * cols;
    const T* dr = dy + r * cols;
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> px = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
      Pack<T, VEC> pd = *reinterpret_cast<const Pack<T, VEC>*>(dr + c);
      Pack<T, VEC> pg = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float xhat = (to_float(px.v[k]) - mu) * rs;
        const float d = to_float(pd.v[k]);
        const float dg = d * to_float(pg.v[k]);
        s1 += dg * xhat;
        s2 += dg;
        atomicAdd(&acc[c + k], d * xhat);
        atomicAdd(&acc[cols + c + k], d);
      }
    }
    s1 = warp_sum(s1) / cols;
    s2 = rms ? 0.f : warp_sum(s2) / cols;       // no centring: the mean term of the gradient vanishes
    T* dxr = dx + r * cols;
    for (int c = lane * VEC; c < cols; c += 32 * VEC) {
      Pack<T, VEC> px = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
      Pack<T, VEC> pd = *reinterpret_cast<const Pack<T, VEC>*>(dr + c);
      Pack<T, VEC> pg = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float xhat = (to_float(px.v[k]) - mu) * rs;
        const float dg = to_float(pd.v[k]) * to_float(pg.v[k]);
        px.v[k] = from_float<T>(rs * (dg - s2 - xhat * s1));
      }
      *reinterpret_cast<Pack<T, VEC>*>(dxr + c) = px;
    }
  }
  __syncthreads();
  float* out = partial + int64_t(blockIdx.x) * 2 * cols;
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) out[c] = acc[c];
}

// Same, for rows of at most 32 * MAXV * VEC elements: every lane owns fixed columns, so
// the weight / bias gradients accumulate in registers across the rows a warp visits and
// meet in shared memory once at the end (no per-element atomics).  The row's operands stay
// packed (16-bit) in registers between the two passes, which keeps the kernel at two CTAs
// per SM; all loads of a row are issued before the first use.
template <typename T, int MAXV>
__global__ void __launch_bounds__(kLnWarps * 32, 2)
layernorm_bwd_reg_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                         const float* __restrict__ mean, const float* __restrict__ rstd, int64_t rows, int cols,
                         T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dres, int rms) {
  constexpr int VEC = 16 / sizeof(T);
  extern __shared__ float acc[];          // [2][cols]
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) acc[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  float dg_acc[MAXV][VEC], db_acc[MAXV][VEC];
  Pack<T, VEC> pg[MAXV];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < cols) pg[j] = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      dg_acc[j][k] = 0.f;
      db_acc[j][k] = 0.f;
      if (c >= cols) pg[j].v[k] = from_float<T>(0.f);
    }
  }
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + (threadIdx.x >> 5); r < rows; r += stride) {
    const T* xr = x + r * cols;
    const T* dr = dy + r * cols;
    Pack<T, VEC> px[MAXV], pd[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) {
        px[j] = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
        pd[j] = *reinterpret_cast<const Pack<T, VEC>*>(dr + c);
      }
    }
    // Ask for the next row of this warp (and this row's residual gradient) now: a warp holds one
    // row at a time, so without this every row would pay the full memory latency.
    {
      const int64_t rn = r + stride;
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int c = (j * 32 + lane) * VEC;
        if (c < cols) {
          if (dres != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(dres + r * cols + c));
          if (rn < rows) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(x + rn * cols + c));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(dy + rn * cols + c));
          }
        }
      }
    }
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const float xh = (to_float(px[j].v[k]) - mu) * rs;
          const float d = to_float(pd[j].v[k]);
          const float dg = d * to_float(pg[j].v[k]);
          s1 += dg * xh;
          s2 += dg;
          dg_acc[j][k] += d * xh;
          db_acc[j][k] += d;
        }
      }
    }
    s1 = warp_sum(s1) / cols;
    s2 = rms ? 0.f : warp_sum(s2) / cols;
    T* dxr = dx + r * cols;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) {
        // `dres`: gradient that reaches the normalised tensor on a second path (the residual
        // stream); adding it here saves the separate accumulation pass.
        Pack<T, VEC> po, pr;
        if (dres != nullptr) pr = *reinterpret_cast<const Pack<T, VEC>*>(dres + r * cols + c);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const float xh = (to_float(px[j].v[k]) - mu) * rs;
          const float dg = to_float(pd[j].v[k]) * to_float(pg[j].v[k]);
          float out = rs * (dg - s2 - xh * s1);
          if (dres != nullptr) out += to_float(pr.v[k]);
          po.v[k] = from_float<T>(out);
        }
        *reinterpret_cast<Pack<T, VEC>*>(dxr + c) = po;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < cols) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        atomicAdd(&acc[c + k], dg_acc[j][k]);
        atomicAdd(&acc[cols + c + k], db_acc[j][k]);
      }
    }
  }
  __syncthreads();
  float* out = partial + int64_t(blockIdx.x) * 2 * cols;
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) out[c] = acc[c];
}

// Backward with a row split over several warps: every thread owns ONE 16-byte pack of a row (its
// columns are fixed for the whole kernel, so the weight / bias gradients still accumulate in
// registers), `tpr` threads (a multiple of 32) cover a row and a CTA works on `rpc` rows at a time.
// About 40 registers per thread instead of 128: four to five times as many rows in flight per SM as
// the one-row-per-warp kernel, whose rate was set by the latency of that loop, not by HBM.  The two
// row statistics cross the row's warps through shared memory (one CTA barrier per iteration,
// buffers alternating so that a fast warp never overwrites what a slow one still reads).
constexpr int kLnSplitThreads = 384;

// Element pair `j` of a 16-byte pack as two fp32 values, and back.  The arithmetic of the kernel
// below runs on such pairs (f32x2 instructions: two elements per issue slot), which is what
// keeps it bound by memory instead of by instruction issue.
template <typename T, int VEC>
__device__ __forceinline__ float2 pack_pair(const Pack<T, VEC>& p, int j) {
  if constexpr (std::is_same<T, float>::value) {
    return make_float2(p.v[2 * j], p.v[2 * j + 1]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(&p)[j];
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    return __half22float2(reinterpret_cast<const __half2*>(&p)[j]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void set_pack_pair(Pack<T, VEC>& p, int j, float2 v) {
  if constexpr (std::is_same<T, float>::value) {
    p.v[2 * j] = v.x;
    p.v[2 * j + 1] = v.y;
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    reinterpret_cast<__nv_bfloat162*>(&p)[j] = __floats2bfloat162_rn(v.x, v.y);
  } else {
    reinterpret_cast<__half2*>(&p)[j] = __floats2half2_rn(v.x, v.y);
  }
}

template <typename T>
__global__ void __launch_bounds__(kLnSplitThreads, 3)
layernorm_bwd_split_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                           const float* __restrict__ mean, const float* __restrict__ rstd, int64_t rows, int cols,
                           T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dres, int rms,
                           int tpr, int rpc) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int PAIRS = VEC / 2;
  constexpr int kWarps = kLnSplitThreads / 32;
  extern __shared__ float acc[];          // [2][cols] gradient sums, then [2][kWarps][2] row statistics
  float* red = acc + 2 * cols;
  for (int i = threadIdx.x; i < 2 * cols; i += blockDim.x) acc[i] = 0.f;
  const int slot = threadIdx.x / tpr;
  const int c = (threadIdx.x - slot * tpr) * VEC;
  const bool col_ok = slot < rpc && c < cols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpr = tpr >> 5;
  Pack<T, VEC> pg;
  float2 dg_acc[PAIRS], db_acc[PAIRS];
#pragma unroll
  for (int k = 0; k < VEC; ++k) pg.v[k] = from_float<T>(0.f);
#pragma unroll
  for (int j = 0; j < PAIRS; ++j) {
    dg_acc[j] = make_float2(0.f, 0.f);
    db_acc[j] = make_float2(0.f, 0.f);
  }
  if (col_ok) pg = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
  __syncthreads();
  const float inv_cols = 1.f / cols;
  int parity = 0;
  for (int64_t r0 = int64_t(blockIdx.x) * rpc; r0 < rows; r0 += int64_t(gridDim.x) * rpc, parity ^= 1) {
    const int64_t r = r0 + slot;
    const bool ok = col_ok && r < rows;
    Pack<T, VEC> px, pd;
    float rs = 0.f, nmurs = 0.f;          // xhat = x * rs + nmurs
    float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
    if (ok) {
      px = *reinterpret_cast<const Pack<T, VEC>*>(x + r * cols + c);
      pd = *reinterpret_cast<const Pack<T, VEC>*>(dy + r * cols + c);
      // Needed only after the barrier: ask for the line now, load it there (four registers less).
      if (dres != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(dres + r * cols + c));
      rs = rstd[r];
      nmurs = -mean[r] * rs;
      const float2 rs2 = make_float2(rs, rs), nm2 = make_float2(nmurs, nmurs);
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const float2 xh = __ffma2_rn(pack_pair(px, j), rs2, nm2);
        const float2 d = pack_pair(pd, j);
        const float2 dg = __fmul2_rn(d, pack_pair(pg, j));
        s1 = __ffma2_rn(dg, xh, s1);
        s2 = __fadd2_rn(s2, dg);
        dg_acc[j] = __ffma2_rn(d, xh, dg_acc[j]);
        db_acc[j] = __fadd2_rn(db_acc[j], d);
      }
    }
    const float w1 = warp_sum(s1.x + s1.y);
    const float w2 = warp_sum(s2.x + s2.y);
    float* mine = red + (parity * kWarps + warp) * 2;
    if (lane == 0) { mine[0] = w1; mine[1] = w2; }
    __syncthreads();
    if (ok) {
      const float* row_red = red + (parity * kWarps + slot * wpr) * 2;
      float t1 = 0.f, t2 = 0.f;
      for (int w = 0; w < wpr; ++w) { t1 += row_red[2 * w]; t2 += row_red[2 * w + 1]; }
      t1 *= inv_cols;
      t2 = rms ? 0.f : t2 * inv_cols;
      // dx = rs * (dg - t2 - xhat * t1) [+ dres]
      const float2 rs2 = make_float2(rs, rs), nm2 = make_float2(nmurs, nmurs);
      const float2 nt1 = make_float2(-t1, -t1), nt2 = make_float2(-t2, -t2);
      Pack<T, VEC> po, pr;
      if (dres != nullptr) pr = *reinterpret_cast<const Pack<T, VEC>*>(dres + r * cols + c);
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const float2 xh = __ffma2_rn(pack_pair(px, j), rs2, nm2);
        const float2 dg = __ffma2_rn(pack_pair(pd, j), pack_pair(pg, j), nt2);     // dg - t2
        float2 out = __fmul2_rn(__ffma2_rn(xh, nt1, dg), rs2);
        if (dres != nullptr) out = __fadd2_rn(out, pack_pair(pr, j));
        set_pack_pair(po, j, out);
      }
      *reinterpret_cast<Pack<T, VEC>*>(dx + r * cols + c) = po;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
      atomicAdd(&acc[c + 2 * j], dg_acc[j].x);
      atomicAdd(&acc[c + 2 * j + 1], dg_acc[j].y);
      atomicAdd(&acc[cols + c + 2 * j], db_acc[j].x);
      atomicAdd(&acc[cols + c + 2 * j + 1], db_acc[j].y);
    }
  }
  __syncthreads();
  float* out = partial + int64_t(blockIdx.x) * 2 * cols;
  for (int i = threadIdx.x; i < 2 * cols; i += blockDim.x) out[i] = acc[i];
}

// Forward for rows of at most 32 * MAXV * VEC elements: the row is read once and stays in
// registers between the statistics and the normalisation; weight and bias are loaded once per warp.
template <typename T, int MAXV>
__global__ void __launch_bounds__(kLnWarps * 32)
layernorm_fwd_reg_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                         int64_t rows, int cols, float eps, T* __restrict__ y, float* __restrict__ mean_out,
                         float* __restrict__ rstd_out, const T* __restrict__ res, const T* __restrict__ res_bias,
                         T* __restrict__ sum_out, int rms) {
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  Pack<T, VEC> pg[MAXV], pb[MAXV];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < cols) {
      pg[j] = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
      if (beta != nullptr) {
        pb[j] = *reinterpret_cast<const Pack<T, VEC>*>(beta + c);
      } else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) pb[j].v[k] = from_float<T>(0.f);
      }
    }
  }
  const float inv_cols = 1.f / cols;
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t r = int64_t(blockIdx.x) * kLnWarps + (threadIdx.x >> 5); r < rows; r += stride) {
    const T* xr = x + r * cols;
    Pack<T, VEC> px[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) px[j] = *reinterpret_cast<const Pack<T, VEC>*>(xr + c);
    }
    {
      const int64_t rn = r + stride;   // next row of this warp: have it in L1 when its turn comes
      if (rn < rows) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = (j * 32 + lane) * VEC;
          if (c < cols) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(x + rn * cols + c));
            if (res != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(res + rn * cols + c));
          }
        }
      }
    }
    if (res != nullptr) {
      // Residual add fused in: the sum (rounded to the storage type, as a separate add would
      // leave it) is written out and normalised.
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int c = (j * 32 + lane) * VEC;
        if (c < cols) {
          const Pack<T, VEC> pr = *reinterpret_cast<const Pack<T, VEC>*>(res + r * cols + c);
          if (res_bias != nullptr) {
            // A per-column vector that belongs to `res` (the bias of the layer that produced it):
            // re-read per row, it stays in L1 and costs no registers between rows.
            const Pack<T, VEC> pv = *reinterpret_cast<const Pack<T, VEC>*>(res_bias + c);
#pragma unroll
            for (int k = 0; k < VEC / 2; ++k)
              set_pack_pair(px[j], k, __fadd2_rn(__fadd2_rn(pack_pair(px[j], k), pack_pair(pr, k)), pack_pair(pv, k)));
          } else {
#pragma unroll
            for (int k = 0; k < VEC / 2; ++k)
              set_pack_pair(px[j], k, __fadd2_rn(pack_pair(px[j], k), pack_pair(pr, k)));
          }
          *reinterpret_cast<Pack<T, VEC>*>(sum_out + r * cols + c) = px[j];
        }
      }
    }
    // Statistics and normalisation on packed fp32 pairs (two elements per instruction).
    float2 s2 = make_float2(0.f, 0.f), ss2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) {
#pragma unroll
        for (int k = 0; k < VEC / 2; ++k) {
          const float2 v = pack_pair(px[j], k);
          s2 = __fadd2_rn(s2, v);
          ss2 = __ffma2_rn(v, v, ss2);
        }
      }
    }
    const float s = warp_sum(s2.x + s2.y);
    const float ss = warp_sum(ss2.x + ss2.y);
    const float mean = rms ? 0.f : s * inv_cols;
    const float rstd = rsqrtf(fmaxf(ss * inv_cols - mean * mean, 0.f) + eps);
    if (lane == 0) { mean_out[r] = mean; rstd_out[r] = rstd; }
    T* yr = y + r * cols;
    const float2 rs2 = make_float2(rstd, rstd), nm2 = make_float2(-mean * rstd, -mean * rstd);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < cols) {
        Pack<T, VEC> po;
#pragma unroll
        for (int k = 0; k < VEC / 2; ++k) {
          const float2 xh = __ffma2_rn(pack_pair(px[j], k), rs2, nm2);          // (x - mean) * rstd
          set_pack_pair(po, k, __ffma2_rn(xh, pack_pair(pg[j], k), pack_pair(pb[j], k)));
        }
        *reinterpret_cast<Pack<T, VEC>*>(yr + c) = po;
      }
    }
  }
}

// dgamma / dbeta = column sums of the per-CTA partials: 32 columns x 8 partial lanes per CTA.
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_bwd_reduce_kernel(const float* __restrict__ partial, int num_partials, int cols,
                            T* __restrict__ dgamma, T* __restrict__ dbeta) {
  __shared__ float red[8][33];
  const int col_lane = threadIdx.x & 31, part_lane = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + col_lane;
  float s = 0.f;
  if (c < 2 * cols) {
    // Four independent loads in flight per thread: the loop is a chain of dependent latencies otherwise.
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int p = part_lane;
    for (; p + 24 < num_partials; p += 32) {
      s += partial[int64_t(p) * 2 * cols + c];
      s1 += partial[int64_t(p + 8) * 2 * cols + c];
      s2 += partial[int64_t(p + 16) * 2 * cols + c];
      s3 += partial[int64_t(p + 24) * 2 * cols + c];
    }
    for (; p < num_partials; p += 8) s += partial[int64_t(p) * 2 * cols + c];
    s += s1 + s2 + s3;
  }
  red[part_lane][col_lane] = s;
  __syncthreads();
  if (part_lane == 0 && c < 2 * cols) {
#pragma unroll
    for (int l = 1; l < 8; ++l) s += red[l][col_lane];
    if (c < cols) dgamma[c] = from_float<T>(s); else dbeta[c - cols] = from_float<T>(s);
  }
}

// ---------------------------------------------------------------------------
// Column sums of a [rows, cols] matrix (bias gradients): every CTA owns a strip of 32 * VEC
// columns and a slice of rows; a warp reads 32 consecutive 16-byte groups of one row, eight
// row lanes accumulate in registers, partial sums meet in `partial[slices][cols]`, and a
// second kernel adds the slices (deterministic, no atomics).
// ---------------------------------------------------------------------------
constexpr int kColsumRowLanes = 8;

template <typename T>
__global__ void __launch_bounds__(32 * kColsumRowLanes)
colsum_partial_kernel(const T* __restrict__ x, int64_t rows, int cols, float* __restrict__ partial) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float red[kColsumRowLanes][32 * VEC + 1];
  const int group = threadIdx.x & 31, row_lane = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + group) * VEC;
  const int64_t per = (rows + gridDim.y - 1) / gridDim.y;
  const int64_t r0 = int64_t(blockIdx.y) * per, r1 = min(rows, r0 + per);
  float acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
  if (c < cols) {
    int64_t r = r0 + row_lane;
    // Four rows in flight per thread.
    for (; r + 3 * kColsumRowLanes < r1; r += 4 * kColsumRowLanes) {
      Pack<T, VEC> p[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        p[u] = *reinterpret_cast<const Pack<T, VEC>*>(x + (r + u * kColsumRowLanes) * cols + c);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] += to_float(p[u].v[k]);
    }
    for (; r < r1; r += kColsumRowLanes) {
      const Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(x + r * cols + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] += to_float(p.v[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < VEC; ++k) red[row_lane][group * VEC + k] = acc[k];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * VEC; i += blockDim.x) {
    const int col = blockIdx.x * 32 * VEC + i;
    if (col < cols) {
      float s = 0.f;
#pragma unroll
      for (int l = 0; l < kColsumRowLanes; ++l) s += red[l][i];
      partial[int64_t(blockIdx.y) * cols + col] = s;
    }
  }
}

template <typename T>
__global__ void colsum_reduce_kernel(const float* __restrict__ partial, int slices, int cols, T* __restrict__ out) {
  // 32 columns x 8 slice lanes per CTA, four loads in flight per thread (same order of additions on every run).
  __shared__ float red[8][33];
  const int col_lane = threadIdx.x & 31, part_lane = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + col_lane;
  float s = 0.f;
  if (c < cols) {
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int p = part_lane;
    for (; p + 24 < slices; p += 32) {
      s += partial[int64_t(p) * cols + c];
      s1 += partial[int64_t(p + 8) * cols + c];
      s2 += partial[int64_t(p + 16) * cols + c];
      s3 += partial[int64_t(p + 24) * cols + c];
    }
    for (; p < slices; p += 8) s += partial[int64_t(p) * cols + c];
    s += s1 + s2 + s3;
  }
  red[part_lane][col_lane] = s;
  __syncthreads();
  if (part_lane == 0 && c < cols) {
#pragma unroll
    for (int l = 1; l < 8; ++l) s += red[l][col_lane];
    out[c] = from_float<T>(s);
  }
}

template <typename T>
bool launch_layernorm_fwd(const T* x, const T* gamma, const T* beta, int64_t rows, int cols, float eps, T* y,
                          float* mean, float* rstd, const T* res, const T* res_bias, T* sum_out, int rms, int sms,
                          cudaStream_t stream) {
  constexpr int kVec = 16 / sizeof(T);
  const int grid = max(1, min(ceil_div(rows, kLnWarps), sms * 6));
  const int packs = ceil_div(cols, 32 * kVec);
  switch (packs) {
    case 1: layernorm_fwd_reg_kernel<T, 1><<<grid, kLnWarps * 32, 0, stream>>>(x, gamma, beta, rows, cols, eps, y, mean, rstd, res, res_bias, sum_out, rms); break;
    case 2: layernorm_fwd_reg_kernel<T, 2><<<grid, kLnWarps * 32, 0, stream>>>(x, gamma, beta, rows, cols, eps, y, mean, rstd, res, res_bias, sum_out, rms); break;
    case 3: layernorm_fwd_reg_kernel<T, 3><<<grid, kLnWarps * 32, 0, stream>>>(x, gamma, beta, rows, cols, eps, y, mean, rstd, res, res_bias, sum_out, rms); break;
    case 4: layernorm_fwd_reg_kernel<T, 4><<<grid, kLnWarps * 32, 0, stream>>>(x, gamma, beta, rows, cols, eps, y, mean, rstd, res, res_bias, sum_out, rms); break;
    default:
      if (res != nullptr) return false;   // the wide-row kernel has no fused add
      layernorm_fwd_kernel<T><<<max(1, min(ceil_div(rows, kLnWarps), sms * 2)), kLnWarps * 32, 0, stream>>>(
          x, gamma, beta, rows, cols, eps, y, mean, rstd, rms);
  }
  return true;
}

template <typename T>
bool launch_layernorm_bwd(const T* dy, const T* x, const T* gamma, const float* mean, const float* rstd, int64_t rows,
                          int cols, T* dx, float* partial, const T* dres, int rms, int grid, size_t smem,
                          cudaStream_t stream) {
  constexpr int kVec = 16 / sizeof(T);
  const int packs = ceil_div(cols, 32 * kVec);
  switch (packs) {
    case 1: layernorm_bwd_reg_kernel<T, 1><<<grid, kLnWarps * 32, smem, stream>>>(dy, x, gamma, mean, rstd, rows, cols, dx, partial, dres, rms); break;
    case 2: layernorm_bwd_reg_kernel<T, 2><<<grid, kLnWarps * 32, smem, stream>>>(dy, x, gamma, mean, rstd, rows, cols, dx, partial, dres, rms); break;
    case 3: layernorm_bwd_reg_kernel<T, 3><<<grid, kLnWarps * 32, smem, stream>>>(dy, x, gamma, mean, rstd, rows, cols, dx, partial, dres, rms); break;
    case 4: layernorm_bwd_reg_kernel<T, 4><<<grid, kLnWarps * 32, smem, stream>>>(dy, x, gamma, mean, rstd, rows, cols, dx, partial, dres, rms); break;
    default:
      if (dres != nullptr) return false;
      layernorm_bwd_kernel<T><<<grid, kLnWarps * 32, smem, stream>>>(dy, x, gamma, mean, rstd, rows, cols, dx, partial, rms);
  }
  return true;
}

}  // namespace

cudaError_t cross_entropy_fwd(DType type, const void* logits, const int64_t* targets, int64_t rows, int64_t vocab,
                              float* lse, float* loss, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(type, T, {
    cross_entropy_fwd_kernel<T><<<static_cast<unsigned>(rows), kCeThreads, 0, stream>>>(
        static_cast<const T*>(logits), targets, vocab, lse, loss);
  })
  return cudaGetLastError();
}

cudaError_t cross_entropy_bwd(DType type, void* logits, const int64_t* targets, const float* lse,
                              const float* scale_ptr, float scale_mul, int64_t rows, int64_t vocab,
                              cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(type, T, {
    cross_entropy_bwd_kernel<T><<<static_cast<unsigned>(rows), kCeThreads, 0, stream>>>(
        static_cast<T*>(logits), targets, lse, scale_ptr, scale_mul, vocab);
  })
  return cudaGetLastError();
}

cudaError_t cross_entropy_fused(DType type, void* logits, const int64_t* targets, float scale, int64_t rows,
                                int64_t vocab, float* loss, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(type, T, {
    cross_entropy_fused_kernel<T><<<static_cast<unsigned>(rows), kCeThreads, 0, stream>>>(
        static_cast<T*>(logits), targets, vocab, scale, loss);
  })
  return cudaGetLastError();
}

// Upper bound of the CTAs any backward path launches (= rows of `partial` the caller allocates).
int layernorm_grid(int64_t rows, int sms) { return max(1, min(ceil_div(rows, 1), sms * 6)); }

bool layernorm_fusable(DType type, int cols) {
  const int vec = type == kF32 ? 4 : 8;
  return cols % vec == 0 && cols <= 32 * 4 * vec;
}

cudaError_t layernorm_fwd(DType type, const void* x, const void* gamma, const void* beta, int64_t rows, int cols,
                          float eps, void* y, float* mean, float* rstd, const void* res, const void* res_bias,
                          void* sum_out, bool rms, int sms, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(type, T, {
    if (cols % (16 / sizeof(T)) != 0) return cudaErrorInvalidValue;
    if (!launch_layernorm_fwd<T>(static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta),
                                 rows, cols, eps, static_cast<T*>(y), mean, rstd, static_cast<const T*>(res),
                                 static_cast<const T*>(res_bias), static_cast<T*>(sum_out), rms ? 1 : 0, sms, stream))
      return cudaErrorInvalidValue;
  })
  return cudaGetLastError();
}

cudaError_t layernorm_bwd(DType type, const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, int64_t rows, int cols, void* dx, void* dgamma, void* dbeta,
                          float* partial, const void* dres, bool rms, int sms, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  int grid = max(1, min(ceil_div(rows, kLnWarps), sms * 2));
  const size_t smem = size_t(2) * cols * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  MB_SWITCH_FLOAT(type, T, {
    constexpr int kVec = 16 / sizeof(T);
    if (cols % kVec != 0) return cudaErrorInvalidValue;
    // Rows that a few warps cover with one pack per thread take the split kernel.
    const int tpr = ceil_div(cols / kVec, 32) * 32;
    static const bool split_off = std::getenv("MB200_LN_SPLIT") != nullptr && std::getenv("MB200_LN_SPLIT")[0] == '0';
    if (tpr <= kLnSplitThreads && !split_off) {
      const int rpc = kLnSplitThreads / tpr;
      grid = max(1, min(ceil_div(rows, rpc), sms * 3));   // three CTAs per SM are resident: one wave
      const size_t smem2 = smem + size_t(2) * (kLnSplitThreads / 32) * 2 * sizeof(float);
      layernorm_bwd_split_kernel<T><<<grid, kLnSplitThreads, smem2, stream>>>(
          static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(gamma), mean, rstd, rows, cols,
          static_cast<T*>(dx), partial, static_cast<const T*>(dres), rms ? 1 : 0, tpr, rpc);
    } else if (!launch_layernorm_bwd<T>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(gamma),
                                 mean, rstd, rows, cols, static_cast<T*>(dx), partial, static_cast<const T*>(dres),
                                 rms ? 1 : 0, grid, smem, stream))
      return cudaErrorInvalidValue;
    layernorm_bwd_reduce_kernel<T><<<ceil_div(2 * cols, 32), 256, 0, stream>>>(
        partial, grid, cols, static_cast<T*>(dgamma), static_cast<T*>(dbeta));
  })
  return cudaGetLastError();
}

int colsum_slices(int64_t rows, int cols, int elem_size, int sms) {
  const int strips = ceil_div(cols, 32 * (16 / elem_size));
  int64_t want = (int64_t(sms) * 4) / strips;
  const int64_t cap = (rows + 63) / 64;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return int(want);
}

cudaError_t column_sum(DType type, const void* x, int64_t rows, int cols, void* out, float* partial, int slices,
                       cudaStream_t stream) {
  if (cols == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(type, T, {
    constexpr int kVec = 16 / sizeof(T);
    if (cols % kVec != 0) return cudaErrorInvalidValue;
    const dim3 grid(ceil_div(cols, 32 * kVec), slices);
    colsum_partial_kernel<T><<<grid, 32 * kColsumRowLanes, 0, stream>>>(static_cast<const T*>(x), rows, cols, partial);
    colsum_reduce_kernel<T><<<ceil_div(cols, 32), 256, 0, stream>>>(partial, slices, cols, static_cast<T*>(out));
  })
  return cudaGetLastError();
}

}  // namespace mb
