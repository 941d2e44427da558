// PyTorch-facing host code of the extension: argument checks, output allocation,
// TMA tensor maps and calls into the torch-free kernel launchers of kernels.h.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kernels.h"

namespace mb {

namespace {

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

#define MB_CHECK_CUDA(t) TORCH_CHECK((t).is_cuda(), #t " must be a CUDA tensor")
#define MB_CHECK_CONTIG(t) TORCH_CHECK((t).is_contiguous(), #t " must be contiguous")
#define MB_CUDA_OK(expr) C10_CUDA_CHECK(expr)

// Number of kernels of this extension enqueued so far by this process.
std::atomic<int64_t> g_launches{0};
#define MB_LAUNCHED(n) g_launches.fetch_add((n), std::memory_order_relaxed)

int sm_count() {
  return at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
}

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

DType float_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return kF32;
    case at::kHalf: return kF16;
    case at::kBFloat16: return kBF16;
    default: TORCH_CHECK(false, "expected float32 / float16 / bfloat16, got ", t);
  }
}

DType int_code(at::ScalarType t) {
  switch (t) {
    case at::kShort: return kI16;
    case at::kInt: return kI32;
    case at::kLong: return kI64;
    default: TORCH_CHECK(false, "expected int16 / int32 / int64, got ", t);
  }
}

int bits_for(int64_t values) {
  int bits = 1;
  while ((int64_t(1) << bits) < values) ++bits;
  return bits;
}

struct SortScratch {
  at::Tensor partial, totals;
  int chunk, num_chunks;
};

SortScratch make_scratch(int64_t n, int nbins, const at::TensorOptions& opts) {
  SortScratch s;
  s.chunk = sort_warp_chunk(n);
  s.num_chunks = std::max<int>(1, int(ceil_div(n, s.chunk)));
  s.partial = at::empty({int64_t(nbins) * s.num_chunks}, opts.dtype(at::kInt));
  s.totals = at::empty({nbins}, opts.dtype(at::kInt));
  return s;
}

void check_index(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kInt && t.dim() == 1, name,
              " must be a contiguous 1-D int32 CUDA tensor");
}

void check_weights(const c10::optional<at::Tensor>& weights, const at::Tensor& x, int64_t copies) {
  if (!weights.has_value()) return;
  TORCH_CHECK(weights->is_cuda() && weights->is_contiguous() && weights->numel() == copies,
              "weights must be a contiguous CUDA tensor with one entry per routed copy");
  TORCH_CHECK(weights->scalar_type() == x.scalar_type(), "weights must have the dtype of x");
}

const void* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// A device counter added to every sequence number of a launch (see EpLayout::seq_base); null when absent.
const int* seq_base_ptr(const c10::optional<at::Tensor>& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->numel() >= 1, "seq_base must be a CUDA int32 tensor");
  return t->data_ptr<int>();
}

at::Tensor build_inverse(const at::Tensor& indices, const at::Tensor& bins, const at::Tensor& padded_bins,
                         int capacity) {
  const int n = int(indices.numel());
  // `indices` is a permutation of the copies, so the kernel writes every entry (-1 for a copy
  // that no bin holds or that exceeds the capacity): no fill beforehand.
  at::Tensor inverse = at::empty({n}, indices.options());
  if (n == 0) return inverse;
  MB_CUDA_OK(inverse_map(indices.data_ptr<int>(), bins.data_ptr<int>(), padded_bins.data_ptr<int>(),
                         int(bins.numel()), n, capacity, inverse.data_ptr<int>(), stream()));
  MB_LAUNCHED(1);
  return inverse;
}

}  // namespace

// ---------------------------------------------------------------------------
// sort / route plan
// ---------------------------------------------------------------------------
std::vector<at::Tensor> sort_pairs(const at::Tensor& x, int64_t end_bit) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 1, "sort expects a 1-D tensor");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = x.numel();
  at::Tensor keys_a = at::empty_like(x), vals_a = at::empty_like(x);
  if (n == 0) return {keys_a, vals_a};
  at::Tensor keys_b = at::empty_like(x), vals_b = at::empty_like(x);
  const DType code = int_code(x.scalar_type());
  const int width = int(x.element_size()) * 8;
  const int total_bits = std::min<int>(std::max<int>(int(end_bit), 1), width);
  const int passes = (total_bits + 7) / 8;
  SortScratch s = make_scratch(n, 256, x.options());
  const void* src_k = x.data_ptr();
  const void* src_v = nullptr;
  void* dst_k[2] = {keys_a.data_ptr(), keys_b.data_ptr()};
  void* dst_v[2] = {vals_a.data_ptr(), vals_b.data_ptr()};
  // Arrange the ping-pong so the last pass lands in (keys_a, vals_a).
  int which = (passes % 2 == 1) ? 0 : 1;
  for (int p = 0; p < passes; ++p) {
    const int shift = p * 8;
    const int bits = std::min(8, total_bits - shift);
    const bool flip = (shift + bits == width);
    MB_CUDA_OK(sort_pass(code, src_k, src_v, n, shift, bits, flip, s.chunk, s.num_chunks,
                         s.partial.data_ptr<int>(), s.totals.data_ptr<int>(), dst_k[which], dst_v[which], nullptr,
                         nullptr, nullptr, 0, 1, stream()));
    MB_LAUNCHED(3);
    src_k = dst_k[which];
    src_v = dst_v[which];
    which ^= 1;
  }
  return {keys_a, vals_a};
}

std::vector<at::Tensor> route_plan(const at::Tensor& top_experts, int64_t num_experts, int64_t block) {
  MB_CHECK_CUDA(top_experts); MB_CHECK_CONTIG(top_experts);
  TORCH_CHECK(top_experts.dim() == 1, "route_plan expects flattened expert ids");
  TORCH_CHECK(num_experts >= 1 && block >= 1, "bad route_plan arguments");
  c10::cuda::CUDAGuard guard(top_experts.device());
  const int64_t n = top_experts.numel();
  auto iopts = top_experts.options().dtype(at::kInt);
  at::Tensor indices = at::empty({n}, iopts), bin_ids = at::empty({n}, iopts);
  if (n == 0) {
    at::Tensor zero = at::zeros({num_experts}, iopts);
    return {indices, bin_ids, zero, zero.clone(), zero.clone()};
  }
  // The scan kernel of the sort writes all three per-expert arrays in full.
  at::Tensor bins = at::empty({num_experts}, iopts), padded_bins = at::empty({num_experts}, iopts);
  at::Tensor tpe = at::empty({num_experts}, iopts);
  // torch.topk yields int64 ids: narrow once, then a single counting-sort pass.
  at::Tensor e32 = top_experts.scalar_type() == at::kInt ? top_experts : top_experts.to(at::kInt);
  if (num_experts <= kMaxSortBins) {
    const int bits = bits_for(num_experts);
    SortScratch s = make_scratch(n, 1 << bits, top_experts.options());
    MB_CUDA_OK(sort_pass(kI32, e32.data_ptr(), nullptr, n, 0, bits, false, s.chunk, s.num_chunks,
                         s.partial.data_ptr<int>(), s.totals.data_ptr<int>(), bin_ids.data_ptr(),
                         indices.data_ptr(), tpe.data_ptr<int>(), bins.data_ptr<int>(),
                         padded_bins.data_ptr<int>(), int(num_experts), int(block), stream()));
    MB_LAUNCHED(3);
    return {indices, bin_ids, bins, padded_bins, tpe};
  }
  // More than 1024 experts: generic multi-pass sort, then histogram and scans.
  auto sorted = sort_pairs(e32, bits_for(num_experts));
  at::Tensor counts = at::bincount(e32, {}, num_experts).to(at::kInt);
  at::Tensor padded = at::floor_divide(counts + (block - 1), block) * block;
  return {sorted[1], sorted[0], at::cumsum(counts, 0).to(at::kInt), at::cumsum(padded, 0).to(at::kInt), counts};
}

// ---------------------------------------------------------------------------
// histogram / cumsum / topology / replicate
// ---------------------------------------------------------------------------
at::Tensor histogram_op(const at::Tensor& x, int64_t num_bins) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 2, "histogram expects [batch, n]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = x.size(0), n = x.size(1);
  at::Tensor out = at::zeros({batch, num_bins}, x.options().dtype(at::kInt));
  if (n == 0 || batch == 0) return out;
  MB_CUDA_OK(histogram(int_code(x.scalar_type()), x.data_ptr(), batch, n, int(num_bins), out.data_ptr<int>(),
                       sm_count(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor cumsum_op(const at::Tensor& x, bool exclusive) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 2, "cumsum expects a 2-D tensor");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty_like(x);
  if (x.numel() == 0) return out;
  MB_CUDA_OK(cumsum(int_code(x.scalar_type()), x.data_ptr(), out.data_ptr(), x.size(0), x.size(1), exclusive,
                    stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor topology_op(const at::Tensor& padded_bins, int64_t block_size, int64_t rows, int64_t cols) {
  check_index(padded_bins, "padded_bins");
  c10::cuda::CUDAGuard guard(padded_bins.device());
  at::Tensor out = at::empty({rows * cols}, padded_bins.options().dtype(at::kShort));
  if (out.numel() == 0) return out;
  MB_CUDA_OK(topology(padded_bins.data_ptr<int>(), int(padded_bins.numel()), int(block_size), int(rows), int(cols),
                      out.data_ptr<int16_t>(), sm_count(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor replicate_forward(const at::Tensor& x, const at::Tensor& bins, int64_t num_outputs) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  check_index(bins, "bins");
  TORCH_CHECK(x.dim() == 2 && x.size(1) == bins.numel(), "replicate expects x[batch, num_bins]");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({x.size(0), num_outputs}, x.options());
  if (out.numel() == 0) return out;
  MB_CUDA_OK(replicate_fwd(int(x.element_size()), x.data_ptr(), bins.data_ptr<int>(), int(bins.numel()), x.size(0),
                           num_outputs, out.data_ptr(), sm_count(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor replicate_backward(const at::Tensor& grad, const at::Tensor& bins) {
  MB_CHECK_CUDA(grad); MB_CHECK_CONTIG(grad);
  check_index(bins, "bins");
  c10::cuda::CUDAGuard guard(grad.device());
  const int num_bins = int(bins.numel());
  at::Tensor out = at::empty({grad.size(0), num_bins}, grad.options());
  if (out.numel() == 0) return out;
  MB_CUDA_OK(replicate_bwd(float_code(grad.scalar_type()), grad.data_ptr(), bins.data_ptr<int>(), num_bins,
                           grad.size(0), grad.size(1), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

// ---------------------------------------------------------------------------
// permutation
// ---------------------------------------------------------------------------
at::Tensor gather_rows_op(const at::Tensor& x, const at::Tensor& indices, const at::Tensor& bin_ids,
                          const c10::optional<at::Tensor>& weights, const at::Tensor& bins,
                          const at::Tensor& padded_bins, int64_t top_k, int64_t out_rows) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 2, "gather expects x[tokens, hidden]");
  check_index(indices, "indices"); check_index(bins, "bins"); check_index(padded_bins, "padded_bins");
  check_weights(weights, x, indices.numel());
  (void)bin_ids;
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({out_rows, x.size(1)}, x.options());
  if (out.numel() == 0) return out;
  MB_CUDA_OK(gather_rows(float_code(x.scalar_type()), x.data_ptr(), indices.data_ptr<int>(), opt_ptr(weights),
                         bins.data_ptr<int>(), padded_bins.data_ptr<int>(), int(bins.numel()), int(top_k), out_rows,
                         int(x.size(1)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor scatter_rows_op(const at::Tensor& x, const at::Tensor& indices, const at::Tensor& bin_ids,
                           const c10::optional<at::Tensor>& weights, const at::Tensor& bins,
                           const at::Tensor& padded_bins, int64_t top_k, int64_t tokens) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 2, "scatter expects x[rows, hidden]");
  check_index(indices, "indices"); check_index(bins, "bins"); check_index(padded_bins, "padded_bins");
  check_weights(weights, x, indices.numel());
  (void)bin_ids;
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({tokens, x.size(1)}, x.options());
  if (out.numel() == 0) return out;
  at::Tensor inverse = build_inverse(indices, bins, padded_bins, -1);
  MB_CUDA_OK(combine_rows(float_code(x.scalar_type()), x.data_ptr(), inverse.data_ptr<int>(), opt_ptr(weights),
                          int(top_k), tokens, int(x.size(1)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor scatter_wgrad_op(const at::Tensor& x, const at::Tensor& grad, const at::Tensor& indices,
                            const at::Tensor& bin_ids, const at::Tensor& bins, const at::Tensor& padded_bins,
                            int64_t top_k) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x); MB_CHECK_CUDA(grad); MB_CHECK_CONTIG(grad);
  TORCH_CHECK(x.scalar_type() == grad.scalar_type() && x.size(1) == grad.size(1), "x / grad mismatch");
  check_index(indices, "indices"); check_index(bins, "bins"); check_index(padded_bins, "padded_bins");
  (void)bin_ids;
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t copies = indices.numel();
  at::Tensor out = at::empty({copies}, x.options());
  if (copies == 0) return out;
  at::Tensor inverse = build_inverse(indices, bins, padded_bins, -1);
  MB_CUDA_OK(scatter_wgrad(float_code(x.scalar_type()), x.data_ptr(), grad.data_ptr(), inverse.data_ptr<int>(),
                           int(top_k), copies, int(x.size(1)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

// Binned layout [E, capacity, h]: the padded gather with uniform padded bins
// (e + 1) * capacity; copies past the capacity have no destination row.
at::Tensor binned_gather_rows(const at::Tensor& x, const at::Tensor& indices,
                              const c10::optional<at::Tensor>& weights, const at::Tensor& bins, int64_t capacity,
                              int64_t top_k) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  check_index(indices, "indices"); check_index(bins, "bins");
  check_weights(weights, x, indices.numel());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t experts = bins.numel();
  at::Tensor out = at::empty({experts, capacity, x.size(1)}, x.options());
  if (out.numel() == 0) return out;
  at::Tensor uniform = (at::arange(1, experts + 1, bins.options().dtype(at::kLong)) * capacity).to(at::kInt);
  MB_CUDA_OK(gather_rows(float_code(x.scalar_type()), x.data_ptr(), indices.data_ptr<int>(), opt_ptr(weights),
                         bins.data_ptr<int>(), uniform.data_ptr<int>(), int(experts), int(top_k),
                         experts * capacity, int(x.size(1)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor binned_scatter_rows(const at::Tensor& x, const at::Tensor& indices,
                               const c10::optional<at::Tensor>& weights, const at::Tensor& bins, int64_t top_k,
                               int64_t tokens) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 3, "binned_scatter expects x[experts, capacity, hidden]");
  check_index(indices, "indices"); check_index(bins, "bins");
  check_weights(weights, x, indices.numel());
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({tokens, x.size(2)}, x.options());
  if (out.numel() == 0) return out;
  at::Tensor inverse = build_inverse(indices, bins, bins, int(x.size(1)));
  MB_CUDA_OK(combine_rows(float_code(x.scalar_type()), x.data_ptr(), inverse.data_ptr<int>(), opt_ptr(weights),
                          int(top_k), tokens, int(x.size(2)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

at::Tensor binned_scatter_wgrad(const at::Tensor& x, const at::Tensor& grad, const at::Tensor& indices,
                                const at::Tensor& bins, int64_t top_k) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x); MB_CHECK_CUDA(grad); MB_CHECK_CONTIG(grad);
  TORCH_CHECK(x.dim() == 3 && x.scalar_type() == grad.scalar_type() && x.size(2) == grad.size(1),
              "x / grad mismatch");
  check_index(indices, "indices"); check_index(bins, "bins");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t copies = indices.numel();
  at::Tensor out = at::empty({copies}, x.options());
  if (copies == 0) return out;
  at::Tensor inverse = build_inverse(indices, bins, bins, int(x.size(1)));
  MB_CUDA_OK(scatter_wgrad(float_code(x.scalar_type()), x.data_ptr(), grad.data_ptr(), inverse.data_ptr<int>(),
                           int(top_k), copies, int(x.size(2)), out.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return out;
}

// ---------------------------------------------------------------------------
// router
// ---------------------------------------------------------------------------
std::vector<at::Tensor> router_topk_forward(const at::Tensor& logits, int64_t top_k, double norm_p) {
  MB_CHECK_CUDA(logits); MB_CHECK_CONTIG(logits);
  TORCH_CHECK(logits.dim() == 2, "router_topk expects logits[tokens, experts]");
  const int64_t tokens = logits.size(0), num_experts = logits.size(1);
  TORCH_CHECK(num_experts <= kRouterMaxExperts && top_k >= 1 && top_k <= kRouterMaxTopK && top_k <= num_experts,
              "router_topk supports up to 1024 experts and top_k <= 8");
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor scores = at::empty_like(logits);
  at::Tensor weights = at::empty({tokens, top_k}, logits.options());
  at::Tensor experts = at::empty({tokens, top_k}, logits.options().dtype(at::kLong));
  if (tokens == 0) return {scores, weights, experts};
  MB_CUDA_OK(router_topk_fwd(float_code(logits.scalar_type()), logits.data_ptr(), tokens, int(num_experts),
                             int(top_k), float(norm_p), scores.data_ptr(), weights.data_ptr(),
                             experts.data_ptr<int64_t>(), stream()));
  MB_LAUNCHED(1);
  return {scores, weights, experts};
}

at::Tensor router_topk_backward(const at::Tensor& scores, const at::Tensor& weights, const at::Tensor& experts,
                                const at::Tensor& dscores, const at::Tensor& dweights, double norm_p) {
  MB_CHECK_CUDA(scores); MB_CHECK_CONTIG(scores); MB_CHECK_CONTIG(dscores); MB_CHECK_CONTIG(dweights);
  MB_CHECK_CONTIG(experts);
  (void)weights;
  TORCH_CHECK(dscores.scalar_type() == scores.scalar_type() && dweights.scalar_type() == scores.scalar_type(),
              "router gradients must have the dtype of the scores");
  const int64_t tokens = scores.size(0), num_experts = scores.size(1), top_k = experts.size(1);
  c10::cuda::CUDAGuard guard(scores.device());
  at::Tensor dlogits = at::empty_like(scores);
  if (tokens == 0) return dlogits;
  MB_CUDA_OK(router_topk_bwd(float_code(scores.scalar_type()), scores.data_ptr(), experts.data_ptr<int64_t>(),
                             dscores.data_ptr(), dweights.data_ptr(), tokens, int(num_experts), int(top_k),
                             float(norm_p), dlogits.data_ptr(), stream()));
  MB_LAUNCHED(1);
  return dlogits;
}

// ---------------------------------------------------------------------------
// grouped GEMM
// ---------------------------------------------------------------------------
namespace {

constexpr int64_t kMaxScatterSegmentsHost = 512;   // = kMaxScatterSegments of the kernel

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result));
    TORCH_CHECK(result == cudaDriverEntryPointSuccess && ptr != nullptr, "cuTensorMapEncodeTiled is unavailable");
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Row-major [rows, cols] 16-bit tensor, box = box_rows x 64 columns, 128-byte swizzle.
CUtensorMap make_tensor_map(const void* base, bool bf16, int64_t rows, int64_t cols, int box_rows) {
  TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "grouped_gemm operands must be 16-byte aligned");
  TORCH_CHECK(cols % 8 == 0, "grouped_gemm operands need a row length that is a multiple of 8 elements");
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(std::max<int64_t>(rows, 1))};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult rc = encode_tiled_fn()(
      &map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
      dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", int(rc));
  return map;
}

// Row-major [rows, cols] 16-bit output, box = 32 x 32, 64-byte swizzle (the epilogue's staging layout).
bool make_output_map(CUtensorMap* map, const void* base, bool bf16, int64_t rows, int64_t cols) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || cols % 8 != 0 || rows < 1) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {32u, 32u};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult rc = encode_tiled_fn()(
      map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
      strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

at::Tensor& status_word(const at::Device& device) {
  // Leaked on purpose: freeing CUDA tensors during static destruction races with
  // the teardown of the CUDA context.
  static auto* words = new std::vector<at::Tensor>(64);
  const int idx = device.index();
  if (!(*words)[idx].defined()) (*words)[idx] = at::zeros({4}, at::TensorOptions().device(device).dtype(at::kInt));
  return (*words)[idx];
}

// MB200_GEMM_TMA_STORE=0 keeps every output store on the LSU path.
bool store_tma_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("MB200_GEMM_TMA_STORE");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return on;
}

// [CTA][16] cycle counters written by builds with -DMB_GEMM_TIMING (zero otherwise).
at::Tensor& timing_words(const at::Device& device) {
  static auto* words = new std::vector<at::Tensor>(64);
  const int idx = device.index();
  if (!(*words)[idx].defined())
    (*words)[idx] = at::zeros({1024, 16}, at::TensorOptions().device(device).dtype(at::kLong));
  return (*words)[idx];
}

}  // namespace

at::Tensor gemm_role_timers(const at::Tensor& like) { return timing_words(like.device()); }

// True when the tcgen05 kernel can run this problem; the Python caller falls back
// to per-group library matmuls otherwise (odd sizes, fp32 inputs).
bool grouped_gemm_supported(const at::Tensor& a, const at::Tensor& b, bool trans_a, bool trans_b,
                            int64_t num_groups) {
  if (!(a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf)) return false;
  if (a.scalar_type() != b.scalar_type() || num_groups > gemm::kMaxGroups || num_groups < 1) return false;
  if (a.dim() != 2) return false;
  if (trans_a) {
    if (b.dim() != 2 || a.size(0) != b.size(0)) return false;
    const int64_t M = a.size(1), N = b.size(1);
    return M % 8 == 0 && N % 8 == 0 && M >= 64 && N >= 64;
  }
  if (b.dim() != 3 || b.size(0) != num_groups) return false;
  const int64_t K = a.size(1);
  const int64_t N = trans_b ? b.size(1) : b.size(2);
  const int64_t Kb = trans_b ? b.size(2) : b.size(1);
  return K == Kb && K % 8 == 0 && N % 8 == 0 && N >= 64 && K >= 8;
}

std::vector<at::Tensor> grouped_gemm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& bins, bool trans_a,
                                     bool trans_b, int64_t epilogue, int64_t act,
                                     const c10::optional<at::Tensor>& aux1, const c10::optional<at::Tensor>& aux2,
                                     bool want_out2, bool want_out3, int64_t num_groups,
                                     const c10::optional<at::Tensor>& c_in, bool zero_tail,
                                     const c10::optional<at::Tensor>& wait_flags, int64_t wait_count,
                                     int64_t wait_stride, int64_t wait_seq, int64_t rows_hint, int64_t pair_mode,
                                     const c10::optional<std::vector<at::Tensor>>& scatter,
                                     const std::vector<int64_t>& scatter_args, double alpha,
                                     const c10::optional<at::Tensor>& a2, const c10::optional<at::Tensor>& b2,
                                     const c10::optional<at::Tensor>& sqnorm,
                                     const c10::optional<at::Tensor>& seq_base) {
  using namespace gemm;
  MB_CHECK_CUDA(a); MB_CHECK_CUDA(b); MB_CHECK_CUDA(bins);
  MB_CHECK_CONTIG(a); MB_CHECK_CONTIG(b); MB_CHECK_CONTIG(bins);
  TORCH_CHECK(bins.scalar_type() == at::kInt && bins.dim() == 1 && bins.numel() == num_groups,
              "bins must be int32 with one entry per group");
  TORCH_CHECK(grouped_gemm_supported(a, b, trans_a, trans_b, num_groups), "unsupported grouped_gemm problem");
  c10::cuda::CUDAGuard guard(a.device());
  const bool bf16 = a.scalar_type() == at::kBFloat16;
  const int layout = trans_a ? kTN : (trans_b ? kNT : kNN);

  GemmParams p{};
  p.bins = bins.data_ptr<int>();
  p.num_groups = int(num_groups);
  p.rows_total = int(a.size(0));
  at::Tensor c;
  if (layout == kTN) {
    p.M = int(a.size(1));
    p.N = int(b.size(1));
    p.K = 0;
    c = c_in.has_value() ? *c_in : at::empty({num_groups, p.M, p.N}, a.options());
  } else {
    p.K = int(a.size(1));
    p.N = int(trans_b ? b.size(1) : b.size(2));
    p.M = 0;
    // With the fused combine the rows go to the peers' return buffers: no local output exists.
    if (scatter.has_value()) c = at::empty({0, p.N}, a.options());
    else c = c_in.has_value() ? *c_in : at::empty({a.size(0), p.N}, a.options());
  }
  TORCH_CHECK(c.is_contiguous() && c.scalar_type() == a.scalar_type(), "bad output buffer");
  const int64_t out_numel = scatter.has_value() ? a.size(0) * int64_t(p.N) : c.numel();
  auto check_aux = [&](const c10::optional<at::Tensor>& t, const char* name) {
    TORCH_CHECK(t.has_value() && t->is_cuda() && t->is_contiguous() && t->numel() == out_numel &&
                    t->scalar_type() == a.scalar_type(),
                name, " must match the output in shape and dtype");
  };
  at::Tensor out2, out3;
  p.epilogue = int(epilogue);
  p.act = int(act);
  p.alpha = float(alpha);
  p.seq_base = seq_base_ptr(seq_base);
  if (sqnorm.has_value()) {
    TORCH_CHECK(layout == kTN && pair_mode != 1 && sqnorm->is_cuda() && sqnorm->scalar_type() == at::kFloat &&
                    sqnorm->numel() >= 1,
                "sqnorm: a CUDA float32 accumulator, weight-gradient (TN) launches of the single-CTA kernel only");
    p.sqnorm = sqnorm->data_ptr<float>();
  }
  if (epilogue == kEpiDAct || epilogue == kEpiGlu || epilogue == kEpiDGlu || epilogue == kEpiAdd) {
    check_aux(aux1, "aux1");
    p.aux1 = aux1->data_ptr();
  }
  if (epilogue == kEpiDGlu) {
    check_aux(aux2, "aux2");
    p.aux2 = aux2->data_ptr();
  }
  if (epilogue != kEpiNone && epilogue != kEpiAdd && want_out2) {
    out2 = at::empty_like(c);
    p.out2 = out2.data_ptr();
  }
  if ((epilogue == kEpiDGlu && want_out3) || epilogue == kEpiGluDual) {
    out3 = at::empty_like(c);
    p.out3 = out3.data_ptr();
  }
  const bool dual = epilogue == kEpiGluDual;
  const bool concat = a2.has_value();
  if (dual) {
    TORCH_CHECK(layout == kNT && b2.has_value() && !a2.has_value() && !scatter.has_value() && p.N >= 128 && pair_mode != 1,
                "the dual-B GLU epilogue needs the NT layout, a second weight tensor and at least 128 output columns");
    TORCH_CHECK(b2->is_cuda() && b2->is_contiguous() && b2->sizes() == b.sizes() && b2->scalar_type() == b.scalar_type(),
                "b2 must match b");
  }
  if (concat) {
    TORCH_CHECK(layout == kNN && b2.has_value() && (epilogue == kEpiNone || epilogue == kEpiAdd),
                "a concatenated contraction needs the NN layout, a2 and b2, and a plain or add epilogue");
    TORCH_CHECK(a2->is_cuda() && a2->is_contiguous() && a2->sizes() == a.sizes() && a2->scalar_type() == a.scalar_type() &&
                    b2->is_cuda() && b2->is_contiguous() && b2->sizes() == b.sizes() && b2->scalar_type() == b.scalar_type(),
                "a2 / b2 must match a / b");
  }
  p.c = c.data_ptr();
  p.status = status_word(a.device()).data_ptr<int>();
#ifdef MB_GEMM_TIMING
  p.timing = reinterpret_cast<long long*>(timing_words(a.device()).data_ptr<int64_t>());
#endif
  p.zero_tail = zero_tail ? 1 : 0;
  {
    static const int diag = [] {
      const char* v = std::getenv("MB200_GEMM_DIAG");
      return v != nullptr ? std::atoi(v) : 0;
    }();
    p.diag = diag;
    static const int band = [] {
      const char* v = std::getenv("MB200_GEMM_BAND");
      return v != nullptr ? std::atoi(v) : 0;
    }();
    p.band_n = band;
  }
  if (wait_flags.has_value()) {
    TORCH_CHECK(wait_flags->is_cuda() && wait_flags->scalar_type() == at::kInt && layout != kTN,
                "wait_flags must be a CUDA int32 tensor (NT / NN layouts only)");
    p.wait_flags = wait_flags->data_ptr<int>();
    p.wait_count = int(wait_count);
    p.wait_stride = int(wait_stride);
    p.wait_seq = int(wait_seq);
  }
  if (scatter.has_value()) {
    // scatter = {data heap bases, flag heap bases, kept counts, done[, routed counts]}; scatter_args = {data offset, flag
    // offset, world, rank, experts, seq, rows of the return buffer}.
    TORCH_CHECK(epilogue == kEpiNone || epilogue == kEpiAdd, "the fused combine supports the plain and the add epilogue");
    TORCH_CHECK(layout == kNN && (scatter->size() == 4 || scatter->size() == 5) && scatter_args.size() == 7,
                "the fused combine needs the NN layout, four or five tensors and seven integers");
    const auto& bases = (*scatter)[0];
    const auto& flag_bases = (*scatter)[1];
    const auto& counts = (*scatter)[2];
    const auto& done = (*scatter)[3];
    const int64_t world = scatter_args[2];
    TORCH_CHECK(bases.is_cuda() && bases.scalar_type() == at::kLong && bases.numel() == world &&
                    flag_bases.is_cuda() && flag_bases.scalar_type() == at::kLong && flag_bases.numel() == world &&
                    counts.scalar_type() == at::kInt && counts.numel() == world * scatter_args[4] &&
                    done.scalar_type() == at::kInt && done.numel() >= world,
                "bad fused-combine arguments");
    TORCH_CHECK(num_groups * world <= kMaxScatterSegmentsHost, "fused combine: too many (expert, rank) segments");
    p.scatter_base = reinterpret_cast<const uint64_t*>(bases.data_ptr<int64_t>());
    p.scatter_flag_base = reinterpret_cast<const uint64_t*>(flag_bases.data_ptr<int64_t>());
    p.scatter_counts = counts.data_ptr<int>();
    p.scatter_raw_counts = p.scatter_counts;
    if (scatter->size() == 5) {   // a capacity limit dropped copies: positions at the sources count them too
      const auto& raw = (*scatter)[4];
      TORCH_CHECK(raw.is_cuda() && raw.scalar_type() == at::kInt && raw.numel() == counts.numel(),
                  "bad raw count matrix of the fused combine");
      p.scatter_raw_counts = raw.data_ptr<int>();
    }
    p.scatter_done = done.data_ptr<int>();
    p.scatter_off = scatter_args[0];
    p.scatter_flag_off = scatter_args[1];
    p.scatter_world = int(world);
    p.scatter_rank = int(scatter_args[3]);
    p.scatter_experts = int(scatter_args[4]);
    p.scatter_seq = int(scatter_args[5]);
    p.scatter_rows = int(scatter_args[6]);
    p.zero_tail = 0;   // there is no local output to clear
  }
  if (out_numel == 0) return {c, out2, out3};

  const int block_n = (p.N >= 256 || dual) ? 256 : (p.N >= 128 ? 128 : 64);
  // CTA pairs (cta_group::2, 256-row tiles, six 32 KB stages per CTA) pull a third less operand
  // traffic through L2, but measured back to back against the single-CTA kernel (alternating
  // launches, L2 flushed, medians) they are 0-8 % slower on every shape tried, from 64 ragged groups
  // of 512 rows to 8 groups of 4096 rows with a 14336-deep contraction, in all three layouts.  They
  // are therefore only taken on request.  pair_mode: 1 = whenever the kernel supports the problem,
  // anything else = never.
  (void)rows_hint;
  const bool pair = pair_mode == 1 && block_n == 256 && sm_count() >= 2 && !scatter.has_value() && !dual && !concat;
  if (!scatter.has_value() && store_tma_enabled()) {
    // Full 32-row quarters of a tile leave through the TMA unit (one instruction per chunk).
    const int64_t out_rows = out_numel / p.N;
    bool ok = make_output_map(&p.out_map[0], p.c, bf16, out_rows, p.N);
    if (ok && p.out2) ok = make_output_map(&p.out_map[1], p.out2, bf16, out_rows, p.N);
    if (ok && p.out3) ok = make_output_map(&p.out_map[2], p.out3, bf16, out_rows, p.N);
    p.store_tma = ok ? 1 : 0;
  }
  CUtensorMap ta, tb;
  int64_t tiles_bound;
  const int64_t num_nb = ceil_div(p.N, block_n);
  if (pair) {
    if (layout == kTN) {
      ta = make_tensor_map(a.data_ptr(), bf16, a.size(0), p.M, 64);
      tb = make_tensor_map(b.data_ptr(), bf16, b.size(0), p.N, 64);
      tiles_bound = num_groups * ceil_div(p.M, 2 * kBlockM) * num_nb;
    } else {
      ta = make_tensor_map(a.data_ptr(), bf16, a.size(0), p.K, kBlockM);
      tb = layout == kNT ? make_tensor_map(b.data_ptr(), bf16, num_groups * p.N, p.K, block_n / 2)
                         : make_tensor_map(b.data_ptr(), bf16, num_groups * p.K, p.N, 64);
      tiles_bound = (ceil_div(a.size(0), 2 * kBlockM) + num_groups) * num_nb;
    }
    const int pairs = int(std::max<int64_t>(1, std::min<int64_t>(tiles_bound, sm_count() / 2)));
    MB_CUDA_OK(launch(bf16, layout, block_n, ta, tb, p, 2 * pairs, stream(), true));
    MB_LAUNCHED(1);
    return {c, out2, out3};
  }
  if (layout == kNT) {
    ta = make_tensor_map(a.data_ptr(), bf16, a.size(0), p.K, kBlockM);
    if (dual) {
      tb = make_tensor_map(b.data_ptr(), bf16, num_groups * p.N, p.K, block_n / 2);
      p.b2_map = make_tensor_map(b2->data_ptr(), bf16, num_groups * p.N, p.K, block_n / 2);
      p.dual_b = 1;
      tiles_bound = (ceil_div(a.size(0), kBlockM) + num_groups) * ceil_div(p.N, block_n / 2);
    } else {
      tb = make_tensor_map(b.data_ptr(), bf16, num_groups * p.N, p.K, block_n);
      tiles_bound = (ceil_div(a.size(0), kBlockM) + num_groups) * num_nb;
    }
  } else if (layout == kNN) {
    ta = make_tensor_map(a.data_ptr(), bf16, a.size(0), p.K, kBlockM);
    tb = make_tensor_map(b.data_ptr(), bf16, num_groups * p.K, p.N, 64);
    if (concat) {
      p.a2_map = make_tensor_map(a2->data_ptr(), bf16, a2->size(0), p.K, kBlockM);
      p.b2_map = make_tensor_map(b2->data_ptr(), bf16, num_groups * p.K, p.N, 64);
      p.k_concat = 1;
    }
    tiles_bound = (ceil_div(a.size(0), kBlockM) + num_groups) * num_nb;
  } else {
    ta = make_tensor_map(a.data_ptr(), bf16, a.size(0), p.M, 64);
    tb = make_tensor_map(b.data_ptr(), bf16, b.size(0), p.N, 64);
    tiles_bound = num_groups * ceil_div(p.M, kBlockM) * num_nb;
  }
  const int grid = int(std::max<int64_t>(1, std::min<int64_t>(tiles_bound, sm_count())));
  MB_CUDA_OK(launch(bf16, layout, block_n, ta, tb, p, grid, stream()));
  MB_LAUNCHED(1);
  return {c, out2, out3};
}

// ---------------------------------------------------------------------------
// block-sparse products
// ---------------------------------------------------------------------------
// `a` and `b` are the operands as stored (contiguous, row-major, 16-bit):
//   sdd  a = [M, K] (or [K, M] with a_mn), b = [K, N] with b_mn (or [N, K]); idx0 / idx1 = block row /
//        block column of every stored block; returns the block values [nnz, 128, 128];
//   dsd  a = block values [nnz, 128, 128] (a_mn = the topology is used transposed), b dense as for sdd;
//   dds  a dense as for sdd, b = block values (b_mn = the topology is NOT transposed);
//        idx0 = segment offsets, idx1 = position of every listed block in the value array (optional:
//        absent = the list is in storage order), idx2 = 128-wide slice of the dense operand per block;
//        returns the dense [out_rows, out_cols] product.
at::Tensor bsmm_op(int64_t mode, const at::Tensor& a, bool a_mn, const at::Tensor& b, bool b_mn,
                   const at::Tensor& idx0, const c10::optional<at::Tensor>& idx1,
                   const c10::optional<at::Tensor>& idx2, int64_t out_rows, int64_t out_cols) {
  using namespace bsmm;
  MB_CHECK_CUDA(a); MB_CHECK_CUDA(b); MB_CHECK_CONTIG(a); MB_CHECK_CONTIG(b);
  TORCH_CHECK((a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf) && a.scalar_type() == b.scalar_type(),
              "bsmm: operands must both be bf16 or both fp16");
  auto check_idx = [](const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kInt, name, " must be a contiguous CUDA int32 tensor");
  };
  check_idx(idx0, "bsmm index 0");
  c10::cuda::CUDAGuard guard(a.device());
  const bool bf16 = a.scalar_type() == at::kBFloat16;
  auto as2d = [](const at::Tensor& t) { return t.dim() == 3 ? t.view({t.size(0) * t.size(1), t.size(2)}) : t; };
  const at::Tensor a2 = as2d(a), b2 = as2d(b);
  TORCH_CHECK(a2.dim() == 2 && b2.dim() == 2, "bsmm: operands must be matrices or [nnz, 128, 128] block arrays");

  BsmmParams p{};
  p.mode = int(mode);
  p.status = status_word(a.device()).data_ptr<int>();
  at::Tensor out;
  if (mode == kSdd) {
    TORCH_CHECK(idx1.has_value(), "sdd needs row and column indices");
    check_idx(*idx1, "bsmm index 1");
    const int64_t nnz = idx0.numel();
    TORCH_CHECK(idx1->numel() == nnz, "sdd: row and column index arrays differ in length");
    const int64_t ka = a_mn ? a2.size(0) : a2.size(1), kb = b_mn ? b2.size(0) : b2.size(1);
    TORCH_CHECK(ka == kb, "sdd: contraction lengths differ");
    const int64_t m = a_mn ? a2.size(1) : a2.size(0), n = b_mn ? b2.size(1) : b2.size(0);
    TORCH_CHECK(m % kBlock == 0 && n % kBlock == 0, "sdd: output dimensions must be multiples of 128");
    out = at::empty({nnz, kBlock, kBlock}, a.options());
    p.K = int(ka);
    p.row_indices = idx0.data_ptr<int>();
    p.column_indices = idx1->data_ptr<int>();
    p.num_tiles = int(nnz);
    p.tiles_inner = 1;
    p.out_ld = kBlock;
    p.out_rows = int(nnz * kBlock);
    p.out_cols = kBlock;
  } else {
    TORCH_CHECK(mode == kDsd || mode == kDds, "bsmm: unknown mode");
    TORCH_CHECK(idx2.has_value(), "dsd / dds need the segment list");
    check_idx(*idx2, "bsmm index 2");
    if (idx1.has_value()) check_idx(*idx1, "bsmm index 1");
    const at::Tensor& values = mode == kDsd ? a2 : b2;
    TORCH_CHECK(values.size(1) == kBlock && values.size(0) % kBlock == 0, "bsmm: block values must be [nnz, 128, 128]");
    TORCH_CHECK(idx2->numel() <= values.size(0) / kBlock && (!idx1.has_value() || idx1->numel() == idx2->numel()),
                "bsmm: the segment list is longer than the block array");
    out = at::empty({out_rows, out_cols}, a.options());
    const int64_t lists = idx0.numel() - 1;
    p.seg_offsets = idx0.data_ptr<int>();
    p.seg_block = idx1.has_value() ? idx1->data_ptr<int>() : nullptr;
    p.seg_k = idx2->data_ptr<int>();
    if (mode == kDsd) {
      TORCH_CHECK(lists * kBlock == out_rows, "dsd: one segment list per 128 output rows expected");
      TORCH_CHECK((b_mn ? b2.size(1) : b2.size(0)) == out_cols, "dsd: dense operand does not match the output width");
      p.tiles_inner = int(ceil_div(out_cols, kBlock));
    } else {
      TORCH_CHECK(lists * kBlock == out_cols, "dds: one segment list per 128 output columns expected");
      TORCH_CHECK((a_mn ? a2.size(1) : a2.size(0)) == out_rows, "dds: dense operand does not match the output height");
      p.tiles_inner = int(ceil_div(out_rows, kBlock));
    }
    p.num_tiles = int(lists * p.tiles_inner);
    p.out_ld = out_cols;
    p.out_rows = int(out_rows);
    p.out_cols = int(out_cols);
  }
  p.out = out.data_ptr();
  if (out.numel() == 0 || p.num_tiles == 0) return out;
  const CUtensorMap ta = make_tensor_map(a2.data_ptr(), bf16, a2.size(0), a2.size(1), a_mn ? 64 : 128);
  const CUtensorMap tb = make_tensor_map(b2.data_ptr(), bf16, b2.size(0), b2.size(1), b_mn ? 64 : 128);
  const int grid = std::max(1, std::min(p.num_tiles, sm_count()));
  MB_CUDA_OK(launch(bf16, a_mn, b_mn, ta, tb, p, grid, stream()));
  MB_LAUNCHED(1);
  return out;
}

// ---------------------------------------------------------------------------
// optimizer
// ---------------------------------------------------------------------------
namespace {

const AdamTensor* table_ptr(const at::Tensor& table) {
  TORCH_CHECK(table.is_cuda() && table.is_contiguous() && table.scalar_type() == at::kByte &&
                  table.numel() % sizeof(AdamTensor) == 0,
              "tensor table must be a contiguous CUDA uint8 tensor of AdamTensor records");
  return reinterpret_cast<const AdamTensor*>(table.data_ptr());
}

const int2* blocks_ptr(const at::Tensor& blocks) {
  TORCH_CHECK(blocks.is_cuda() && blocks.is_contiguous() && blocks.scalar_type() == at::kInt && blocks.dim() == 2 &&
                  blocks.size(1) == 2,
              "block table must be a contiguous CUDA int32 [n, 2] tensor");
  return reinterpret_cast<const int2*>(blocks.data_ptr());
}

DType code_of(int64_t code) {
  TORCH_CHECK(code >= kF32 && code <= kBF16, "bad dtype code");
  return static_cast<DType>(code);
}

}  // namespace

int64_t adam_record_size() { return sizeof(AdamTensor); }

void adam_step_op(const at::Tensor& table, const at::Tensor& blocks, int64_t chunk, int64_t param_code,
                  int64_t grad_code, double lr, double beta1, double beta2, double eps, double weight_decay,
                  double bias1, double bias2, const c10::optional<at::Tensor>& grad_scale,
                  const c10::optional<at::Tensor>& hyper) {
  c10::cuda::CUDAGuard guard(table.device());
  const float* hyper_ptr = nullptr;
  if (hyper.has_value()) {
    TORCH_CHECK(hyper->is_cuda() && hyper->scalar_type() == at::kFloat && hyper->numel() >= 3 && hyper->is_contiguous(),
                "hyper must be three contiguous CUDA float32 values {lr, bias1, bias2}");
    hyper_ptr = hyper->data_ptr<float>();
  }
  const float* scale = nullptr;
  if (grad_scale.has_value()) {
    TORCH_CHECK(grad_scale->is_cuda() && grad_scale->scalar_type() == at::kFloat, "grad_scale must be CUDA float32");
    scale = grad_scale->data_ptr<float>();
  }
  MB_CUDA_OK(adam_step(code_of(param_code), code_of(grad_code), table_ptr(table), blocks_ptr(blocks),
                       int(blocks.size(0)), int(chunk), float(lr), float(beta1), float(beta2), float(eps),
                       float(weight_decay), float(bias1), float(bias2), scale, hyper_ptr, stream()));
  MB_LAUNCHED(1);
}

void grad_sqnorm_op(const at::Tensor& table, const at::Tensor& blocks, int64_t chunk, int64_t grad_code,
                    at::Tensor out_accum) {
  c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(out_accum.is_cuda() && out_accum.scalar_type() == at::kFloat, "accumulator must be CUDA float32");
  MB_CUDA_OK(grad_sqnorm(code_of(grad_code), table_ptr(table), blocks_ptr(blocks), int(blocks.size(0)), int(chunk),
                         out_accum.data_ptr<float>(), stream()));
  MB_LAUNCHED(1);
}

void clip_coeff_op(const at::Tensor& sqnorm, double max_norm, double extra_scale, at::Tensor out) {
  c10::cuda::CUDAGuard guard(sqnorm.device());
  TORCH_CHECK(sqnorm.is_cuda() && sqnorm.scalar_type() == at::kFloat && out.is_cuda() &&
                  out.scalar_type() == at::kFloat && out.numel() >= 2,
              "clip_coeff expects CUDA float32 tensors (out with >= 2 elements)");
  MB_CUDA_OK(clip_coeff(sqnorm.data_ptr<float>(), float(max_norm), float(extra_scale), out.data_ptr<float>(),
                        stream()));
  MB_LAUNCHED(1);
}

// ---------------------------------------------------------------------------
// fused row-wise ops: cross entropy, LayerNorm
// ---------------------------------------------------------------------------
std::vector<at::Tensor> cross_entropy_forward(const at::Tensor& logits, const at::Tensor& targets) {
  MB_CHECK_CUDA(logits); MB_CHECK_CONTIG(logits); MB_CHECK_CUDA(targets); MB_CHECK_CONTIG(targets);
  TORCH_CHECK(logits.dim() == 2 && targets.dim() == 1 && targets.scalar_type() == at::kLong &&
                  targets.numel() == logits.size(0),
              "cross_entropy expects logits[rows, vocab] and int64 targets[rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  auto fopts = logits.options().dtype(at::kFloat);
  at::Tensor lse = at::empty({logits.size(0)}, fopts), loss = at::empty({logits.size(0)}, fopts);
  MB_CUDA_OK(cross_entropy_fwd(float_code(logits.scalar_type()), logits.data_ptr(), targets.data_ptr<int64_t>(),
                               logits.size(0), logits.size(1), lse.data_ptr<float>(), loss.data_ptr<float>(),
                               stream()));
  MB_LAUNCHED(1);
  return {loss, lse};
}

// Overwrites `logits` with its gradient: (softmax - onehot) * scale[0] * scale_mul.
// Per-row loss; `logits` is overwritten with the gradient of `scale * sum(loss)` with respect to it.
at::Tensor cross_entropy_fused_(at::Tensor logits, const at::Tensor& targets, double scale) {
  MB_CHECK_CUDA(logits); MB_CHECK_CONTIG(logits); MB_CHECK_CUDA(targets); MB_CHECK_CONTIG(targets);
  TORCH_CHECK(logits.dim() == 2 && targets.dim() == 1 && targets.size(0) == logits.size(0) &&
                  targets.scalar_type() == at::kLong,
              "cross_entropy expects logits[rows, vocab] and int64 targets[rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  MB_CUDA_OK(cross_entropy_fused(float_code(logits.scalar_type()), logits.data_ptr(), targets.data_ptr<int64_t>(),
                                 float(scale), logits.size(0), logits.size(1), loss.data_ptr<float>(), stream()));
  MB_LAUNCHED(1);
  return loss;
}

void cross_entropy_backward_(at::Tensor logits, const at::Tensor& targets, const at::Tensor& lse,
                             const c10::optional<at::Tensor>& scale, double scale_mul) {
  MB_CHECK_CUDA(logits); MB_CHECK_CONTIG(logits);
  c10::cuda::CUDAGuard guard(logits.device());
  const float* sp = nullptr;
  if (scale.has_value()) {
    TORCH_CHECK(scale->is_cuda() && scale->scalar_type() == at::kFloat && scale->numel() >= 1,
                "scale must be a CUDA float32 scalar");
    sp = scale->data_ptr<float>();
  }
  MB_CUDA_OK(cross_entropy_bwd(float_code(logits.scalar_type()), logits.data_ptr(), targets.data_ptr<int64_t>(),
                               lse.data_ptr<float>(), sp, float(scale_mul), logits.size(0), logits.size(1),
                               stream()));
  MB_LAUNCHED(1);
}

bool layernorm_can_fuse(const at::Tensor& x) {
  return x.is_cuda() && x.dim() == 2 && layernorm_fusable(float_code(x.scalar_type()), int(x.size(1)));
}

// Returns {y, mean, rstd, s}: s = x + res [+ res_bias] (or x itself without res) is the tensor that
// was normalised.
// `beta` absent = RMS norm (no centring, no bias); the returned mean is then all zeros.
std::vector<at::Tensor> layernorm_forward(const at::Tensor& x, const at::Tensor& gamma,
                                          const c10::optional<at::Tensor>& beta, double eps,
                                          const c10::optional<at::Tensor>& res,
                                          const c10::optional<at::Tensor>& res_bias) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x); MB_CHECK_CONTIG(gamma);
  const bool rms = !beta.has_value();
  TORCH_CHECK(x.dim() == 2 && gamma.numel() == x.size(1) && gamma.scalar_type() == x.scalar_type() &&
                  (rms || (beta->is_contiguous() && beta->numel() == x.size(1) &&
                           beta->scalar_type() == x.scalar_type())),
              "layernorm expects x[rows, cols] and weight / bias of length cols in the dtype of x");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  at::Tensor sum = x;
  if (res.has_value()) {
    TORCH_CHECK(res->is_cuda() && res->is_contiguous() && res->sizes() == x.sizes() &&
                    res->scalar_type() == x.scalar_type() && layernorm_can_fuse(x),
                "layernorm: the fused residual needs a tensor like x and rows the register kernel holds");
    sum = at::empty_like(x);
  }
  const void* res_bias_ptr = nullptr;
  if (res_bias.has_value()) {
    TORCH_CHECK(res.has_value() && res_bias->is_cuda() && res_bias->is_contiguous() &&
                    res_bias->numel() == x.size(1) && res_bias->scalar_type() == x.scalar_type(),
                "layernorm: res_bias goes with res and holds one value per column in the dtype of x");
    res_bias_ptr = res_bias->data_ptr();
  }
  auto fopts = x.options().dtype(at::kFloat);
  at::Tensor mean = at::empty({x.size(0)}, fopts), rstd = at::empty({x.size(0)}, fopts);
  MB_CUDA_OK(layernorm_fwd(float_code(x.scalar_type()), x.data_ptr(), gamma.data_ptr(),
                           rms ? nullptr : beta->data_ptr(), x.size(0), int(x.size(1)), float(eps), y.data_ptr(),
                           mean.data_ptr<float>(), rstd.data_ptr<float>(),
                           res.has_value() ? res->data_ptr() : nullptr, res_bias_ptr,
                           res.has_value() ? sum.data_ptr() : nullptr, rms, sm_count(), stream()));
  MB_LAUNCHED(1);
  return {y, mean, rstd, sum};
}

std::vector<at::Tensor> layernorm_backward(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gamma,
                                           const at::Tensor& mean, const at::Tensor& rstd,
                                           const c10::optional<at::Tensor>& dres, bool rms) {
  MB_CHECK_CUDA(dy); MB_CHECK_CONTIG(dy); MB_CHECK_CONTIG(x);
  c10::cuda::CUDAGuard guard(x.device());
  if (dres.has_value())
    TORCH_CHECK(dres->is_cuda() && dres->is_contiguous() && dres->sizes() == x.sizes() &&
                    dres->scalar_type() == x.scalar_type() && layernorm_can_fuse(x),
                "layernorm: the fused gradient add needs a tensor like x and rows the register kernel holds");
  at::Tensor dx = at::empty_like(x), dgamma = at::empty_like(gamma), dbeta = at::empty_like(gamma);
  const int grid = layernorm_grid(x.size(0), sm_count());
  at::Tensor partial = at::empty({grid, 2 * x.size(1)}, x.options().dtype(at::kFloat));
  MB_CUDA_OK(layernorm_bwd(float_code(x.scalar_type()), dy.data_ptr(), x.data_ptr(), gamma.data_ptr(),
                           mean.data_ptr<float>(), rstd.data_ptr<float>(), x.size(0), int(x.size(1)), dx.data_ptr(),
                           dgamma.data_ptr(), dbeta.data_ptr(), partial.data_ptr<float>(),
                           dres.has_value() ? dres->data_ptr() : nullptr, rms, sm_count(), stream()));
  MB_LAUNCHED(2);
  return {dx, dgamma, dbeta};
}

// ---------------------------------------------------------------------------
// load-balancing loss, rotary embedding
// ---------------------------------------------------------------------------
namespace {
LblArgs lbl_args(const std::vector<at::Tensor>& scores, const std::vector<at::Tensor>& counts) {
  TORCH_CHECK(!scores.empty() && scores.size() == counts.size() && scores.size() <= size_t(kLblMaxLayers),
              "load_balancing_loss: between 1 and ", kLblMaxLayers, " layers per call");
  LblArgs args{};
  const auto& first = scores[0];
  for (size_t l = 0; l < scores.size(); ++l) {
    const auto& s = scores[l];
    const auto& c = counts[l];
    TORCH_CHECK(s.is_cuda() && s.is_contiguous() && s.dim() == 2 && s.sizes() == first.sizes() &&
                    s.scalar_type() == first.scalar_type(),
                "load_balancing_loss: scores must be contiguous CUDA [tokens, experts] tensors of one shape and dtype");
    TORCH_CHECK(c.is_cuda() && c.is_contiguous() && c.scalar_type() == at::kInt && c.numel() == s.size(1),
                "load_balancing_loss: counts must be contiguous CUDA int32 [experts] tensors");
    args.scores[l] = s.data_ptr();
    args.counts[l] = c.data_ptr<int>();
  }
  return args;
}
}  // namespace

at::Tensor lbl_forward_op(const std::vector<at::Tensor>& scores, const std::vector<at::Tensor>& counts, double scale) {
  LblArgs args = lbl_args(scores, counts);
  const auto& first = scores[0];
  c10::cuda::CUDAGuard guard(first.device());
  const int layers = int(scores.size());
  const int slices = lbl_slices(first.size(0), layers, sm_count());
  auto fopts = first.options().dtype(at::kFloat);
  at::Tensor partial = at::empty({layers * slices}, fopts), loss = at::empty({}, fopts);
  at::Tensor ticket = at::zeros({1}, first.options().dtype(at::kInt));
  MB_CUDA_OK(lbl_forward(float_code(first.scalar_type()), args, layers, first.size(0), int(first.size(1)), float(scale),
                         partial.data_ptr<float>(), slices, ticket.data_ptr<int>(), loss.data_ptr<float>(), stream()));
  MB_LAUNCHED(1);
  return loss;
}

std::vector<at::Tensor> lbl_backward_op(const std::vector<at::Tensor>& scores, const std::vector<at::Tensor>& counts,
                                        double scale, const at::Tensor& gout) {
  LblArgs args = lbl_args(scores, counts);
  const auto& first = scores[0];
  TORCH_CHECK(gout.is_cuda() && gout.scalar_type() == at::kFloat && gout.numel() == 1, "gout must be a CUDA fp32 scalar");
  c10::cuda::CUDAGuard guard(first.device());
  std::vector<at::Tensor> out;
  for (size_t l = 0; l < scores.size(); ++l) {
    out.push_back(at::empty_like(scores[l]));
    args.dscores[l] = out.back().data_ptr();
  }
  MB_CUDA_OK(lbl_backward(float_code(first.scalar_type()), args, int(scores.size()), first.size(0), int(first.size(1)),
                          float(scale), gout.data_ptr<float>(), sm_count(), stream()));
  MB_LAUNCHED(1);
  return out;
}

// x: [batch, seq, heads, dim] view with unit stride in dim; returns a contiguous tensor of that shape.
at::Tensor rope_op(const at::Tensor& x, const at::Tensor& cosv, const at::Tensor& sinv, bool inverse) {
  MB_CHECK_CUDA(x);
  TORCH_CHECK(x.dim() == 4 && x.stride(3) == 1, "rope expects [batch, seq, heads, dim] with unit stride in dim");
  TORCH_CHECK(cosv.is_cuda() && sinv.is_cuda() && cosv.is_contiguous() && sinv.is_contiguous() &&
                  cosv.scalar_type() == at::kFloat && sinv.scalar_type() == at::kFloat && cosv.dim() == 2 &&
                  cosv.size(0) >= x.size(1) && cosv.size(1) == x.size(3) / 2 && sinv.sizes() == cosv.sizes(),
              "rope expects fp32 cos / sin tables [>= seq, dim / 2]");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "rope: input must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty(x.sizes(), x.options());
  MB_CUDA_OK(rope(float_code(x.scalar_type()), x.data_ptr(), x.stride(0), x.stride(1), x.stride(2),
                  cosv.data_ptr<float>(), sinv.data_ptr<float>(), int(x.size(0)), int(x.size(1)), int(x.size(2)),
                  int(x.size(3)), inverse, out.data_ptr(), sm_count(), stream()));
  MB_LAUNCHED(1);
  return out;
}

// Sum over the rows of x[rows, cols]: the bias gradient of a linear layer.
at::Tensor column_sum_op(const at::Tensor& x) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  TORCH_CHECK(x.dim() == 2 && (x.size(1) * x.element_size()) % 16 == 0,
              "column_sum expects x[rows, cols] with rows of a multiple of 16 bytes");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({x.size(1)}, x.options());
  const int slices = colsum_slices(x.size(0), int(x.size(1)), int(x.element_size()), sm_count());
  at::Tensor partial = at::empty({slices, x.size(1)}, x.options().dtype(at::kFloat));
  if (x.size(0) == 0) return out.zero_();
  MB_CUDA_OK(column_sum(float_code(x.scalar_type()), x.data_ptr(), x.size(0), int(x.size(1)), out.data_ptr(),
                        partial.data_ptr<float>(), slices, stream()));
  MB_LAUNCHED(2);
  return out;
}

// ---------------------------------------------------------------------------
// symmetric heap (CUDA IPC) and expert-parallel exchange
// ---------------------------------------------------------------------------
// Allocates `nbytes` of zeroed device memory that peers can map, and returns it as a
// uint8 tensor together with its IPC handle (a 64-byte CPU uint8 tensor).  The memory
// comes straight from cudaMalloc: IPC handles refer to whole allocations, which rules
// out sub-blocks of the caching allocator.
std::vector<at::Tensor> symm_alloc(int64_t nbytes) {
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&ptr, static_cast<size_t>(nbytes)));
  C10_CUDA_CHECK(cudaMemset(ptr, 0, static_cast<size_t>(nbytes)));
  cudaIpcMemHandle_t handle;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&handle, ptr));
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  at::Tensor local = at::from_blob(
      ptr, {nbytes}, [](void* p) { cudaFree(p); },
      at::TensorOptions().device(at::Device(at::kCUDA, dev)).dtype(at::kByte));
  at::Tensor h = at::empty({static_cast<int64_t>(sizeof(handle))}, at::TensorOptions().dtype(at::kByte));
  std::memcpy(h.data_ptr(), &handle, sizeof(handle));
  return {local, h};
}

// Maps a peer's allocation into this process; returns the device address.
int64_t symm_open(const at::Tensor& handle) {
  TORCH_CHECK(!handle.is_cuda() && handle.scalar_type() == at::kByte &&
                  handle.numel() == static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)),
              "symm_open expects the 64-byte CPU handle produced by symm_alloc");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void symm_close(int64_t ptr) { C10_CUDA_CHECK(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr))); }

namespace {

EpLayout make_layout(const at::Tensor& peer_base, int64_t world, int64_t rank, int64_t num_experts,
                     int64_t experts_per_rank, int64_t capacity_rows, int64_t off_counts, int64_t off_count_flags,
                     const c10::optional<at::Tensor>& seq_base = c10::nullopt) {
  TORCH_CHECK(peer_base.is_cuda() && peer_base.scalar_type() == at::kLong && peer_base.numel() == world,
              "peer_base must be a CUDA int64 tensor with one address per rank");
  EpLayout L;
  L.peer_base = reinterpret_cast<const uint64_t*>(peer_base.data_ptr<int64_t>());
  L.world = int(world);
  L.rank = int(rank);
  L.num_experts = int(num_experts);
  L.experts_per_rank = int(experts_per_rank);
  L.capacity_rows = int(capacity_rows);
  L.off_counts = off_counts;
  L.off_count_flags = off_count_flags;
  L.seq_base = seq_base_ptr(seq_base);
  return L;
}

int* status_ptr(const at::Tensor& t) { return status_word(t.device()).data_ptr<int>(); }

}  // namespace

void ep_exchange_counts_op(const at::Tensor& tpe, const at::Tensor& peer_base, int64_t world, int64_t rank,
                           int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows, int64_t off_counts,
                           int64_t off_count_flags, int64_t seq, int64_t expert_capacity, at::Tensor counts_out,
                           at::Tensor kept_out, at::Tensor recv_bins, at::Tensor scratch,
                           const c10::optional<at::Tensor>& seq_base) {
  check_index(tpe, "tokens_per_expert");
  c10::cuda::CUDAGuard guard(tpe.device());
  TORCH_CHECK(tpe.numel() == num_experts && counts_out.numel() == world * num_experts &&
                  kept_out.numel() == world * num_experts && recv_bins.numel() == experts_per_rank &&
                  counts_out.scalar_type() == at::kInt && kept_out.scalar_type() == at::kInt &&
                  recv_bins.scalar_type() == at::kInt && scratch.scalar_type() == at::kInt && expert_capacity >= 0,
              "bad ep_exchange_counts arguments");
  const EpLayout L = make_layout(peer_base, world, rank, num_experts, experts_per_rank, capacity_rows, off_counts,
                                 off_count_flags, seq_base);
  MB_CUDA_OK(ep_exchange_counts(tpe.data_ptr<int>(), L, int(seq), int(expert_capacity), counts_out.data_ptr<int>(),
                                kept_out.data_ptr<int>(), recv_bins.data_ptr<int>(), scratch.data_ptr<int>(),
                                int(scratch.numel()), status_ptr(tpe), stream()));
  MB_LAUNCHED(1);
}

void ep_push_rows_op(const at::Tensor& x, const at::Tensor& indices, const c10::optional<at::Tensor>& weights,
                     const at::Tensor& bins, const at::Tensor& counts, const at::Tensor& peer_base, int64_t world,
                     int64_t rank, int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows,
                     int64_t off_counts, int64_t off_count_flags, const at::Tensor& data_base, int64_t off_recv,
                     int64_t off_flags, int64_t off_free, int64_t seq, int64_t top_k, at::Tensor done,
                     const c10::optional<at::Tensor>& dropped_rows, const c10::optional<at::Tensor>& seq_base) {
  MB_CHECK_CUDA(x); MB_CHECK_CONTIG(x);
  void* dropped = nullptr;
  if (dropped_rows.has_value()) {
    TORCH_CHECK(dropped_rows->is_cuda() && dropped_rows->is_contiguous() && dropped_rows->scalar_type() == x.scalar_type() &&
                    dropped_rows->dim() == 2 && dropped_rows->size(1) == x.size(1) &&
                    dropped_rows->size(0) >= indices.numel(),
                "dropped_rows must be a [>= copies, hidden] buffer of the activation dtype");
    dropped = dropped_rows->data_ptr();
  }
  check_index(indices, "indices"); check_index(bins, "bins");
  check_weights(weights, x, indices.numel());
  c10::cuda::CUDAGuard guard(x.device());
  const EpLayout L = make_layout(peer_base, world, rank, num_experts, experts_per_rank, capacity_rows, off_counts,
                                 off_count_flags, seq_base);
  TORCH_CHECK(data_base.is_cuda() && data_base.scalar_type() == at::kLong && data_base.numel() == world,
              "data_base must be a CUDA int64 tensor with one address per rank");
  MB_CUDA_OK(ep_push_rows(float_code(x.scalar_type()), x.data_ptr(), indices.data_ptr<int>(), opt_ptr(weights),
                          bins.data_ptr<int>(), counts.data_ptr<int>(), L,
                          reinterpret_cast<const uint64_t*>(data_base.data_ptr<int64_t>()), off_recv, off_flags,
                          off_free, int(seq), int(top_k), int(indices.numel()), int(x.size(1)),
                          done.data_ptr<int>(), status_ptr(x), dropped, sm_count(), stream()));
  MB_LAUNCHED(1);
}

void ep_return_rows_op(const at::Tensor& y, const at::Tensor& counts, const at::Tensor& raw_counts,
                       const at::Tensor& peer_base, int64_t world,
                       int64_t rank, int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows,
                       int64_t off_counts, int64_t off_count_flags, const at::Tensor& data_base, int64_t off_ret,
                       int64_t off_flags, int64_t seq, int64_t ret_rows, at::Tensor done,
                       const c10::optional<at::Tensor>& seq_base) {
  MB_CHECK_CUDA(y); MB_CHECK_CONTIG(y);
  c10::cuda::CUDAGuard guard(y.device());
  const EpLayout L = make_layout(peer_base, world, rank, num_experts, experts_per_rank, capacity_rows, off_counts,
                                 off_count_flags, seq_base);
  TORCH_CHECK(data_base.is_cuda() && data_base.scalar_type() == at::kLong && data_base.numel() == world,
              "data_base must be a CUDA int64 tensor with one address per rank");
  TORCH_CHECK(raw_counts.is_cuda() && raw_counts.scalar_type() == at::kInt && raw_counts.numel() == counts.numel(),
              "raw_counts must match counts");
  MB_CUDA_OK(ep_return_rows(float_code(y.scalar_type()), y.data_ptr(), counts.data_ptr<int>(),
                            raw_counts.data_ptr<int>(), L,
                            reinterpret_cast<const uint64_t*>(data_base.data_ptr<int64_t>()), off_ret, off_flags,
                            int(seq), int(y.size(1)), int(y.size(0)), int(ret_rows), done.data_ptr<int>(),
                            status_ptr(y), sm_count(), stream()));
  MB_LAUNCHED(1);
}

void ep_wait_flags_op(const at::Tensor& flags, int64_t count, int64_t seq, int64_t code,
                      const c10::optional<at::Tensor>& seq_base) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.numel() >= count, "bad flags tensor");
  c10::cuda::CUDAGuard guard(flags.device());
  MB_CUDA_OK(ep_wait_flags(flags.data_ptr<int>(), int(count), int(seq), seq_base_ptr(seq_base), status_ptr(flags),
                           int(code), stream()));
  MB_LAUNCHED(1);
}

void ep_set_flag_op(at::Tensor flag, int64_t value, const c10::optional<at::Tensor>& seq_base) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt && flag.numel() >= 1, "bad flag tensor");
  c10::cuda::CUDAGuard guard(flag.device());
  MB_CUDA_OK(ep_set_flag(flag.data_ptr<int>(), int(value), seq_base_ptr(seq_base), stream()));
  MB_LAUNCHED(1);
}

// Gradient all-reduce / reduce-scatter over peer memory: see dp_comm.cu.  `like` names the device and
// the element type of the gradient buffer that lives at `off_grad` in the symmetric heap.
void dp_allreduce_op(const at::Tensor& like, const at::Tensor& peer_base, int64_t world, int64_t rank,
                     int64_t off_grad, int64_t off_ready, int64_t off_done, int64_t start, int64_t count,
                     int64_t bucket, int64_t seq, double scale, bool scatter_only, at::Tensor ticket, int64_t ctas,
                     const c10::optional<at::Tensor>& seq_base) {
  MB_CHECK_CUDA(like);
  TORCH_CHECK(peer_base.is_cuda() && peer_base.scalar_type() == at::kLong && peer_base.numel() == world,
              "peer_base must be a CUDA int64 tensor with one address per rank");
  TORCH_CHECK(ticket.is_cuda() && ticket.scalar_type() == at::kInt && ticket.numel() >= 1, "bad ticket tensor");
  c10::cuda::CUDAGuard guard(like.device());
  DpLayout L{};
  L.peer_base = reinterpret_cast<const uint64_t*>(peer_base.data_ptr<int64_t>());
  L.world = int(world);
  L.rank = int(rank);
  L.off_grad = off_grad;
  L.off_ready = off_ready;
  L.off_done = off_done;
  L.seq_base = seq_base_ptr(seq_base);
  MB_CUDA_OK(dp_allreduce(float_code(like.scalar_type()), L, start, count, int(bucket), int(seq), float(scale),
                          scatter_only, ticket.data_ptr<int>(), status_ptr(like), int(ctas), stream()));
  MB_LAUNCHED(1);
}

int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// A replayed CUDA graph launches kernels that never pass through the ops above: the owner of the
// graph adds the number it recorded, once per replay.
void count_launches(int64_t n) { MB_LAUNCHED(n); }

// Reads (and optionally clears) the status word of the current device; nonzero means
// a kernel abandoned a wait.  Synchronises the device.
int64_t read_status(bool clear) {
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  at::Tensor& word = status_word(at::Device(at::kCUDA, dev));
  const int64_t value = word[0].item<int>();
  if (clear && value != 0) word.zero_();
  return value;
}

}  // namespace mb
