// Multi-tensor optimizer kernels for sm_100a: fused Adam(W) with fp32 master
// weights and a 16-bit shadow copy, and the squared gradient norm that feeds
// gradient clipping.  One launch covers every parameter tensor of a group: a
// device table lists the tensors, a second table maps each CTA to a (tensor,
// chunk) pair.  The clip coefficient is read from device memory, so the whole
// optimizer step runs without the host ever looking at a value.
//
// The reference has no optimizer (its experiment scripts use Megatron-LM's:
// exp/dmoe/dmoe_125m_8gpu.sh:65-72, bf16 parameters with fp32 main copies, Adam,
// clip-grad 1.0); this is the native equivalent for the stand-alone trainer.
#include "common.cuh"

namespace mb {

namespace {

constexpr int kOptThreads = 256;

template <typename T>
__device__ __forceinline__ void load8f(const T* p, float (&out)[8]) {
  struct alignas(16) Raw { T v[8]; } raw;
  *reinterpret_cast<uint4*>(&raw) = __ldcs(reinterpret_cast<const uint4*>(p));
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_float(raw.v[i]);
}
// Optimizer state is touched once per step: streaming loads and stores keep it from displacing
// anything useful in L2.
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float (&out)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p + 4));
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store8f(T* p, const float (&in)[8]) {
  struct alignas(16) Raw { T v[8]; } raw;
#pragma unroll
  for (int i = 0; i < 8; ++i) raw.v[i] = from_float<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&raw);
}
template <>
__device__ __forceinline__ void store8f<float>(float* p, const float (&in)[8]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(in[0], in[1], in[2], in[3]));
  __stcs(reinterpret_cast<float4*>(p + 4), make_float4(in[4], in[5], in[6], in[7]));
}

// grad_scale_ptr[0] multiplies every gradient (clip coefficient x 1/accumulation).  `hyper`, when
// given, holds {lr, bias1, bias2} in device memory and replaces the arguments of those names: a
// launch recorded in a CUDA graph then follows the schedule without being re-recorded.
template <typename P, typename G>
__global__ void __launch_bounds__(kOptThreads)
adam_kernel(const AdamTensor* __restrict__ tensors, const int2* __restrict__ blocks, int chunk, float lr,
            float beta1, float beta2, float eps, float weight_decay, float bias1, float bias2,
            const float* __restrict__ grad_scale_ptr, const float* __restrict__ hyper) {
  if (hyper != nullptr) {
    lr = hyper[0];
    bias1 = hyper[1];
    bias2 = hyper[2];
  }
  const int2 job = blocks[blockIdx.x];
  const AdamTensor t = tensors[job.x];
  const int64_t begin = int64_t(job.y) * chunk;
  const int64_t end = min(begin + chunk, t.numel);
  const float gscale = grad_scale_ptr != nullptr ? *grad_scale_ptr : 1.f;
  P* param = static_cast<P*>(t.param);
  const G* grad = static_cast<const G*>(t.grad);
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(param) | reinterpret_cast<uintptr_t>(grad)) % 16 == 0) &&
                      ((reinterpret_cast<uintptr_t>(t.master) | reinterpret_cast<uintptr_t>(t.exp_avg) |
                        reinterpret_cast<uintptr_t>(t.exp_avg_sq)) % 16 == 0);
  auto update = [&](float g, float& w, float& m, float& v) {
    g *= gscale;
    m = beta1 * m + (1.f - beta1) * g;
    v = beta2 * v + (1.f - beta2) * g * g;
    const float denom = sqrtf(v / bias2) + eps;
    w = w - lr * ((m / bias1) / denom + weight_decay * w);
  };
  // Chunks start at multiples of the chunk size, so alignment carries over from the base.
  const int64_t vec_end = vec_ok ? begin + ((end - begin) / 8) * 8 : begin;
  // Two independent 8-element batches per iteration: fourteen 16-byte loads in flight per thread.
  int64_t i = begin + int64_t(threadIdx.x) * 8;
  for (; i + kOptThreads * 8 < vec_end; i += 2 * kOptThreads * 8) {
    const int64_t i2 = i + kOptThreads * 8;
    float g[8], w[8], m[8], v[8], g2[8], w2[8], m2[8], v2[8];
    load8f<G>(grad + i, g);
    load8f<float>(t.master + i, w);
    load8f<float>(t.exp_avg + i, m);
    load8f<float>(t.exp_avg_sq + i, v);
    load8f<G>(grad + i2, g2);
    load8f<float>(t.master + i2, w2);
    load8f<float>(t.exp_avg + i2, m2);
    load8f<float>(t.exp_avg_sq + i2, v2);
#pragma unroll
    for (int j = 0; j < 8; ++j) update(g[j], w[j], m[j], v[j]);
    store8f<float>(t.master + i, w);
    store8f<float>(t.exp_avg + i, m);
    store8f<float>(t.exp_avg_sq + i, v);
    store8f<P>(param + i, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) update(g2[j], w2[j], m2[j], v2[j]);
    store8f<float>(t.master + i2, w2);
    store8f<float>(t.exp_avg + i2, m2);
    store8f<float>(t.exp_avg_sq + i2, v2);
    store8f<P>(param + i2, w2);
  }
  for (; i < vec_end; i += kOptThreads * 8) {
    float g[8], w[8], m[8], v[8];
    load8f<G>(grad + i, g);
    load8f<float>(t.master + i, w);
    load8f<float>(t.exp_avg + i, m);
    load8f<float>(t.exp_avg_sq + i, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) update(g[j], w[j], m[j], v[j]);
    store8f<float>(t.master + i, w);
    store8f<float>(t.exp_avg + i, m);
    store8f<float>(t.exp_avg_sq + i, v);
    store8f<P>(param + i, w);
  }
  // Scalar path: unaligned tensors and the (< 8 element) tail.
  for (int64_t j = vec_end + threadIdx.x; j < end; j += kOptThreads) {
    float w = t.master[j], m = t.exp_avg[j], v = t.exp_avg_sq[j];
    update(to_float(grad[j]), w, m, v);
    t.master[j] = w; t.exp_avg[j] = m; t.exp_avg_sq[j] = v;
    param[j] = from_float<P>(w);
  }
}

template <typename G>
__global__ void __launch_bounds__(kOptThreads)
sqnorm_kernel(const AdamTensor* __restrict__ tensors, const int2* __restrict__ blocks, int chunk,
              float* __restrict__ out) {
  __shared__ float warp_sums[kOptThreads / 32];
  const int2 job = blocks[blockIdx.x];
  const AdamTensor t = tensors[job.x];
  const int64_t begin = int64_t(job.y) * chunk;
  const int64_t end = min(begin + chunk, t.numel);
  const G* grad = static_cast<const G*>(t.grad);
  float acc = 0.f;
  const bool vec_ok = reinterpret_cast<uintptr_t>(grad) % 16 == 0;
  const int64_t vec_end = vec_ok ? begin + ((end - begin) / 8) * 8 : begin;
  for (int64_t i = begin + int64_t(threadIdx.x) * 8; i < vec_end; i += kOptThreads * 8) {
    float g[8];
    load8f<G>(grad + i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += g[j] * g[j];
  }
  for (int64_t j = vec_end + threadIdx.x; j < end; j += kOptThreads) {
    const float g = to_float(grad[j]);
    acc += g * g;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kOptThreads / 32 ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    // The weight lets a caller count replicated tensors once across ranks.
    if (threadIdx.x == 0 && v != 0.f) atomicAdd(out, v * t.norm_weight);
  }
}

// coeff = min(1, max_norm / (sqrt(sqnorm) + 1e-6)) * extra_scale, written to out[0]; out[1] = norm.
__global__ void clip_coeff_kernel(const float* __restrict__ sqnorm, float max_norm, float extra_scale,
                                  float* __restrict__ out) {
  const float norm = sqrtf(*sqnorm);
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  if (!isfinite(norm)) c = 0.f;   // a non-finite gradient skips the update instead of poisoning the weights
  out[0] = c * extra_scale;
  out[1] = norm;
}

}  // namespace

cudaError_t adam_step(DType param_type, DType grad_type, const AdamTensor* tensors, const int2* blocks,
                      int num_blocks, int chunk, float lr, float beta1, float beta2, float eps, float weight_decay,
                      float bias1, float bias2, const float* grad_scale, const float* hyper, cudaStream_t stream) {
  if (num_blocks == 0) return cudaSuccess;
#define MB_ADAM(P, G)                                                                                        \
  adam_kernel<P, G><<<num_blocks, kOptThreads, 0, stream>>>(tensors, blocks, chunk, lr, beta1, beta2, eps,   \
                                                            weight_decay, bias1, bias2, grad_scale, hyper)
  if (param_type == kBF16 && grad_type == kBF16) MB_ADAM(__nv_bfloat16, __nv_bfloat16);
  else if (param_type == kF16 && grad_type == kF16) MB_ADAM(__half, __half);
  else if (param_type == kF32 && grad_type == kF32) MB_ADAM(float, float);
  else if (param_type == kBF16 && grad_type == kF32) MB_ADAM(__nv_bfloat16, float);
  else return cudaErrorInvalidValue;
#undef MB_ADAM
  return cudaGetLastError();
}

cudaError_t grad_sqnorm(DType grad_type, const AdamTensor* tensors, const int2* blocks, int num_blocks, int chunk,
                        float* out_accum, cudaStream_t stream) {
  if (num_blocks == 0) return cudaSuccess;
  MB_SWITCH_FLOAT(grad_type, G, { sqnorm_kernel<G><<<num_blocks, kOptThreads, 0, stream>>>(tensors, blocks, chunk, out_accum); })
  return cudaGetLastError();
}

cudaError_t clip_coeff(const float* sqnorm, float max_norm, float extra_scale, float* out, cudaStream_t stream) {
  clip_coeff_kernel<<<1, 1, 0, stream>>>(sqnorm, max_norm, extra_scale, out);
  return cudaGetLastError();
}

}  // namespace mb
