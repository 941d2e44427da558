// Small model-side kernels for sm_100a: the load-balancing loss of all MoE layers in one
// reduction (and its gradient in one broadcast), and rotary position embedding.
//
// Reference behaviour: megablocks/layers/moe.py:39-89 (batched_load_balancing_loss builds the
// concatenated [tokens, layers * experts] score matrix, takes column means and a dot product with
// the concatenated token counts).  Here nothing is concatenated: every CTA reduces a slice of one
// layer's score matrix directly against that layer's counts, partial results are added in a fixed
// order by the last CTA to finish (deterministic), and the backward writes
// d scores[l][t, e] = g * scale * counts[l][e] in one launch over all layers.
#include "common.cuh"

namespace mb {

namespace {

constexpr int kLblThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kLblThreads)
lbl_fwd_kernel(LblArgs a, int64_t tokens, int experts, float scale, float* __restrict__ partial, int* ticket,
               float* __restrict__ loss) {
  const int layer = blockIdx.y, slices = gridDim.x;
  const T* __restrict__ scores = static_cast<const T*>(a.scores[layer]);
  const int* __restrict__ counts = a.counts[layer];
  const int64_t rows_per = (tokens + slices - 1) / slices;
  const int64_t r0 = min(tokens, int64_t(blockIdx.x) * rows_per), r1 = min(tokens, r0 + rows_per);
  // Threads tile (row lanes x columns): a row of scores is read by consecutive threads.
  const int cols_per_pass = min(experts, kLblThreads);
  const int row_lanes = kLblThreads / cols_per_pass;
  const int col_lane = threadIdx.x % cols_per_pass, row_lane = threadIdx.x / cols_per_pass;
  float acc = 0.f;
  if (row_lane < row_lanes) {
    for (int c = col_lane; c < experts; c += cols_per_pass) {
      float colsum = 0.f;
      for (int64_t r = r0 + row_lane; r < r1; r += row_lanes) colsum += to_float(scores[r * experts + c]);
      acc += colsum * float(__ldg(counts + c));
    }
  }
  // Block reduction in a fixed order.
  __shared__ float red[kLblThreads / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < kLblThreads / 32; ++w) total += red[w];
    partial[layer * slices + blockIdx.x] = total;
    __threadfence();
    const int n = gridDim.x * gridDim.y;
    last_s = atomicAdd(ticket, 1) == n - 1;
    if (last_s) {
      *ticket = 0;
      __threadfence();
      float sum = 0.f;
      for (int i = 0; i < n; ++i) sum += *reinterpret_cast<volatile float*>(partial + i);
      *loss = sum * scale;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kLblThreads)
lbl_bwd_kernel(LblArgs a, int64_t tokens, int experts, float scale, const float* __restrict__ gout) {
  const int layer = blockIdx.y;
  T* __restrict__ out = static_cast<T*>(a.dscores[layer]);
  const int* __restrict__ counts = a.counts[layer];
  const float g = *gout * scale;
  constexpr int VEC = 16 / sizeof(T);
  if (experts % VEC == 0) {
    // Every row is the same vector g * counts: each thread builds its 16-byte piece once and
    // stores it down its column strip.
    const int vecs_per_row = experts / VEC;
    const int64_t total = tokens * vecs_per_row;
    const int64_t stride = int64_t(gridDim.x) * kLblThreads;
    int64_t i = int64_t(blockIdx.x) * kLblThreads + threadIdx.x;
    // A stride that is a multiple of the row length keeps a thread in one column strip.
    const bool fixed = stride % vecs_per_row == 0;
    struct alignas(16) Raw { T v[VEC]; } piece;
    int have = -1;
    for (; i < total; i += stride) {
      const int v = int(i % vecs_per_row);
      if (!fixed || have != v) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) piece.v[k] = from_float<T>(g * float(__ldg(counts + v * VEC + k)));
        have = v;
      }
      *reinterpret_cast<uint4*>(out + i * VEC) = *reinterpret_cast<const uint4*>(&piece);
    }
    return;
  }
  const int64_t total = tokens * experts;
  for (int64_t i = int64_t(blockIdx.x) * kLblThreads + threadIdx.x; i < total; i += int64_t(gridDim.x) * kLblThreads)
    out[i] = from_float<T>(g * float(__ldg(counts + int(i % experts))));
}

// ---------------------------------------------------------------------------
// rotary position embedding
// ---------------------------------------------------------------------------
// x is [batch, seq, heads, dim] with arbitrary strides for the first three dimensions (a view into
// the fused QKV projection) and unit stride in dim; out is contiguous.  The pairs (i, i + dim/2)
// are rotated by the angle of (position, i): forward with +sin, `inverse` (the gradient) with -sin.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(const T* __restrict__ x, int64_t sb, int64_t ss, int64_t sh, const float* __restrict__ cosv,
            const float* __restrict__ sinv, int batch, int seq, int heads, int dim, int inverse, T* __restrict__ out) {
  constexpr int VEC = 16 / sizeof(T);
  const int half = dim / 2, vecs = half / VEC;
  const int64_t total = int64_t(batch) * seq * heads * vecs;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int v = int(i % vecs);
    int64_t rest = i / vecs;
    const int h = int(rest % heads);
    rest /= heads;
    const int s = int(rest % seq);
    const int b = int(rest / seq);
    const T* src = x + b * sb + s * ss + h * sh + v * VEC;
    struct alignas(16) Raw { T v[VEC]; } lo, hi, olo, ohi;
    *reinterpret_cast<uint4*>(&lo) = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(&hi) = *reinterpret_cast<const uint4*>(src + half);
    const float* cp = cosv + int64_t(s) * half + v * VEC;
    const float* sp = sinv + int64_t(s) * half + v * VEC;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const float c = __ldg(cp + k), sn = inverse ? -__ldg(sp + k) : __ldg(sp + k);
      const float a1 = to_float(lo.v[k]), a2 = to_float(hi.v[k]);
      olo.v[k] = from_float<T>(a1 * c - a2 * sn);
      ohi.v[k] = from_float<T>(a2 * c + a1 * sn);
    }
    T* dst = out + ((int64_t(b) * seq + s) * heads + h) * dim + v * VEC;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&olo);
    *reinterpret_cast<uint4*>(dst + half) = *reinterpret_cast<const uint4*>(&ohi);
  }
}

}  // namespace

int lbl_slices(int64_t tokens, int layers, int sms) {
  const int64_t want = (2 * sms) / (layers < 1 ? 1 : layers);
  const int64_t cap = (tokens + 255) / 256;
  return int(want < cap ? (want < 1 ? 1 : want) : (cap < 1 ? 1 : cap));
}

cudaError_t lbl_forward(DType type, const LblArgs& args, int layers, int64_t tokens, int experts, float scale,
                        float* partial, int slices, int* ticket, float* loss, cudaStream_t stream) {
  if (layers < 1 || layers > kLblMaxLayers || experts < 1) return cudaErrorInvalidValue;
  const dim3 grid(slices, layers);
  MB_SWITCH_FLOAT(type, T, { lbl_fwd_kernel<T><<<grid, kLblThreads, 0, stream>>>(args, tokens, experts, scale, partial, ticket, loss); })
  return cudaGetLastError();
}

cudaError_t lbl_backward(DType type, const LblArgs& args, int layers, int64_t tokens, int experts, float scale,
                         const float* gout, int sms, cudaStream_t stream) {
  if (layers < 1 || layers > kLblMaxLayers || experts < 1) return cudaErrorInvalidValue;
  if (tokens == 0) return cudaSuccess;
  const int per_layer = max(1, min(ceil_div(tokens * experts, kLblThreads * 8), (4 * sms) / layers + 1));
  const dim3 grid(per_layer, layers);
  MB_SWITCH_FLOAT(type, T, { lbl_bwd_kernel<T><<<grid, kLblThreads, 0, stream>>>(args, tokens, experts, scale, gout); })
  return cudaGetLastError();
}

cudaError_t rope(DType type, const void* x, int64_t stride_b, int64_t stride_s, int64_t stride_h, const float* cosv,
                 const float* sinv, int batch, int seq, int heads, int dim, bool inverse, void* out, int sms,
                 cudaStream_t stream) {
  const int elem = type == kF32 ? 4 : 2;
  const int vec = 16 / elem;
  if (dim % (2 * vec) != 0 || (stride_b * elem) % 16 || (stride_s * elem) % 16 || (stride_h * elem) % 16)
    return cudaErrorInvalidValue;
  const int64_t total = int64_t(batch) * seq * heads * (dim / 2 / vec);
  if (total == 0) return cudaSuccess;
  int64_t blocks = (total + 255) / 256;
  if (blocks > int64_t(sms) * 8) blocks = int64_t(sms) * 8;
  const int grid = int(blocks < 1 ? 1 : blocks);
  MB_SWITCH_FLOAT(type, T, {
    rope_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(x), stride_b, stride_s, stride_h, cosv, sinv,
                                             batch, seq, heads, dim, inverse ? 1 : 0, static_cast<T*>(out));
  })
  return cudaGetLastError();
}

}  // namespace mb
