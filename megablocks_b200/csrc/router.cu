// Router selection kernels for sm_100a: softmax -> top-k -> optional p-norm
// normalisation in one pass over the logits, and the matching backward.
//
// Reference semantics (megablocks/layers/router.py:87-106): scores are the
// softmax of the logits rounded to the logits' dtype; the k largest *rounded*
// scores are selected (ties go to the lowest expert id); weights are optionally
// divided by their p-norm (p = 1 or 2).  One warp owns one token; with at most
// 1024 experts a lane holds at most 32 scores in registers; the kernels are compiled for 1, 2, 4,
// 8, 16 and 32 scores per lane and the launch picks the smallest that covers the expert count, so
// a 64-expert router does not walk 32 mostly empty slots per loop.
#include "common.cuh"

namespace mb {

namespace {

constexpr int kMaxPerLane = kRouterMaxExperts / 32;
constexpr int kMaxTopK = kRouterMaxTopK;

template <typename T, int PL>
__global__ void __launch_bounds__(128)
router_topk_fwd_kernel(const T* __restrict__ logits, int64_t tokens, int num_experts, int top_k, float norm_p,
                       T* __restrict__ scores, T* __restrict__ weights, int64_t* __restrict__ experts) {
  const int lane = threadIdx.x & 31;
  const int64_t t = int64_t(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const T* row = logits + t * num_experts;
  float v[PL];
  float vmax = -INFINITY;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = lane + j * 32;
    v[j] = e < num_experts ? to_float(row[e]) : -INFINITY;
    vmax = fmaxf(vmax, v[j]);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, d));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = lane + j * 32;
    v[j] = e < num_experts ? __expf(v[j] - vmax) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  const float inv = 1.f / sum;
  T* srow = scores + t * num_experts;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = lane + j * 32;
    if (e < num_experts) {
      const T r = from_float<T>(v[j] * inv);
      srow[e] = r;
      v[j] = to_float(r);          // selection runs on the rounded scores
    } else {
      v[j] = -1.f;
    }
  }
  float chosen_w[kMaxTopK];
  int chosen_e[kMaxTopK];
  for (int s = 0; s < top_k; ++s) {
    float best = -2.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PL; ++j) {
      const int e = lane + j * 32;
      if (v[j] > best) { best = v[j]; best_e = e; }   // ascending e within a lane: first wins ties
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    chosen_w[s] = best;
    chosen_e[s] = best_e;
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int j = 0; j < PL; ++j)
        if (j == (best_e >> 5)) v[j] = -1.f;
    }
  }
  if (lane == 0) {
    float norm = 1.f;
    if (norm_p > 0.f) {
      float acc = 0.f;
      for (int s = 0; s < top_k; ++s) acc += (norm_p == 1.f) ? fabsf(chosen_w[s]) : chosen_w[s] * chosen_w[s];
      norm = (norm_p == 1.f) ? acc : sqrtf(acc);
      norm = to_float(from_float<T>(norm));   // the norm is itself a tensor of dtype T
    }
    for (int s = 0; s < top_k; ++s) {
      weights[t * top_k + s] = from_float<T>(norm_p > 0.f ? chosen_w[s] / norm : chosen_w[s]);
      experts[t * top_k + s] = chosen_e[s];
    }
  }
}

// dlogits = s * (g - <g, s>) with g = dscores + scatter(top-k weight grads).
template <typename T, int PL>
__global__ void __launch_bounds__(128)
router_topk_bwd_kernel(const T* __restrict__ scores, const int64_t* __restrict__ experts,
                       const T* __restrict__ dscores, const T* __restrict__ dweights, int64_t tokens,
                       int num_experts, int top_k, float norm_p, T* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int64_t t = int64_t(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const T* srow = scores + t * num_experts;
  const T* grow = dscores + t * num_experts;
  // Gradient with respect to the k selected (pre-normalisation) scores.
  float dsel[kMaxTopK];
  int sel[kMaxTopK];
  float raw[kMaxTopK];
  float norm_acc = 0.f, dot = 0.f;
  for (int s = 0; s < top_k; ++s) {
    sel[s] = static_cast<int>(experts[t * top_k + s]);
    raw[s] = to_float(srow[sel[s]]);
    dsel[s] = to_float(dweights[t * top_k + s]);
    norm_acc += (norm_p == 1.f) ? fabsf(raw[s]) : raw[s] * raw[s];
    dot += dsel[s] * raw[s];
  }
  if (norm_p > 0.f) {
    const float norm = (norm_p == 1.f) ? norm_acc : sqrtf(norm_acc);
    for (int s = 0; s < top_k; ++s) {
      const float dnorm = (norm_p == 1.f) ? (raw[s] >= 0.f ? 1.f : -1.f) : raw[s] / norm;
      dsel[s] = dsel[s] / norm - dot * dnorm / (norm * norm);
    }
  }
  float g[PL];
  float inner = 0.f;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = lane + j * 32;
    float gv = 0.f;
    if (e < num_experts) {
      gv = to_float(grow[e]);
      for (int s = 0; s < top_k; ++s)
        if (sel[s] == e) gv += dsel[s];
      inner += gv * to_float(srow[e]);
    }
    g[j] = gv;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) inner += __shfl_xor_sync(0xffffffffu, inner, d);
  T* drow = dlogits + t * num_experts;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = lane + j * 32;
    if (e < num_experts) drow[e] = from_float<T>(to_float(srow[e]) * (g[j] - inner));
  }
}

}  // namespace

cudaError_t router_topk_fwd(DType type, const void* logits, int64_t tokens, int num_experts, int top_k,
                            float norm_p, void* scores, void* weights, int64_t* experts, cudaStream_t stream) {
  if (num_experts > 32 * kMaxPerLane || top_k < 1 || top_k > kMaxTopK || top_k > num_experts)
    return cudaErrorInvalidValue;
  if (tokens == 0) return cudaSuccess;
#define MB_ROUTER_FWD(PL)                                                                            \
  router_topk_fwd_kernel<T, PL><<<ceil_div(tokens, 4), 128, 0, stream>>>(                            \
      static_cast<const T*>(logits), tokens, num_experts, top_k, norm_p, static_cast<T*>(scores),    \
      static_cast<T*>(weights), experts)
  MB_SWITCH_FLOAT(type, T, {
    if (num_experts <= 32) MB_ROUTER_FWD(1);
    else if (num_experts <= 64) MB_ROUTER_FWD(2);
    else if (num_experts <= 128) MB_ROUTER_FWD(4);
    else if (num_experts <= 256) MB_ROUTER_FWD(8);
    else if (num_experts <= 512) MB_ROUTER_FWD(16);
    else MB_ROUTER_FWD(32);
  })
#undef MB_ROUTER_FWD
  return cudaGetLastError();
}

cudaError_t router_topk_bwd(DType type, const void* scores, const int64_t* experts, const void* dscores,
                            const void* dweights, int64_t tokens, int num_experts, int top_k, float norm_p,
                            void* dlogits, cudaStream_t stream) {
  if (tokens == 0) return cudaSuccess;
  if (num_experts > 32 * kMaxPerLane) return cudaErrorInvalidValue;
#define MB_ROUTER_BWD(PL)                                                                                          \
  router_topk_bwd_kernel<T, PL><<<ceil_div(tokens, 4), 128, 0, stream>>>(                                          \
      static_cast<const T*>(scores), experts, static_cast<const T*>(dscores), static_cast<const T*>(dweights),     \
      tokens, num_experts, top_k, norm_p, static_cast<T*>(dlogits))
  MB_SWITCH_FLOAT(type, T, {
    if (num_experts <= 32) MB_ROUTER_BWD(1);
    else if (num_experts <= 64) MB_ROUTER_BWD(2);
    else if (num_experts <= 128) MB_ROUTER_BWD(4);
    else if (num_experts <= 256) MB_ROUTER_BWD(8);
    else if (num_experts <= 512) MB_ROUTER_BWD(16);
    else MB_ROUTER_BWD(32);
  })
#undef MB_ROUTER_BWD
  return cudaGetLastError();
}

}  // namespace mb
