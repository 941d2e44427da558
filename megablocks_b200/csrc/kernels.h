// Launch interface of the sm_100a kernels: plain pointers, sizes and a stream.
// Every function enqueues work on `stream` and returns cudaGetLastError().
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace mb {

enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2, kI16 = 3, kI32 = 4, kI64 = 5 };

// ---- metadata.cu --------------------------------------------------------------
constexpr int kMaxSortBins = 1024;   // one sort pass handles up to 10 key bits

// Elements a warp owns in the sort passes, and the resulting number of warp chunks.
int sort_warp_chunk(int64_t n);

// One stable counting-sort pass on key bits [shift, shift + bits).  `partial`
// ([2^bits * num_chunks] ints) and `totals` ([2^bits] ints) are scratch.  When
// `tpe` is non-null the pass also writes the per-bin counts, their inclusive prefix
// sums (`bins`) and the block-padded prefix sums (`padded_bins`) for the first
// `num_real_bins` bins.  `vals_in == nullptr` means "values are 0..n-1".
cudaError_t sort_pass(DType key_type, const void* keys, const void* vals_in, int64_t n, int shift, int bits,
                      bool flip_sign, int chunk, int num_chunks, int* partial, int* totals, void* keys_out,
                      void* vals_out, int* tpe, int* bins, int* padded_bins, int num_real_bins, int block,
                      cudaStream_t stream);
cudaError_t histogram(DType type, const void* x, int64_t batch, int64_t n, int num_bins, int* out_zeroed,
                      int sms, cudaStream_t stream);
cudaError_t cumsum(DType type, const void* x, void* out, int64_t rows, int64_t cols, bool exclusive,
                   cudaStream_t stream);
cudaError_t topology(const int* padded_bins, int num_bins, int block_size, int rows, int cols, int16_t* out,
                     int sms, cudaStream_t stream);
cudaError_t replicate_fwd(int elem_size, const void* x, const int* bins, int num_bins, int64_t batch,
                          int64_t num_outputs, void* out, int sms, cudaStream_t stream);
cudaError_t replicate_bwd(DType type, const void* grad, const int* bins, int num_bins, int64_t batch,
                          int64_t num_inputs, void* out, cudaStream_t stream);

// ---- permute.cu ---------------------------------------------------------------
cudaError_t gather_rows(DType type, const void* x, const int* indices, const void* weights, const int* bins,
                        const int* padded_bins, int num_bins, int top_k, int64_t out_rows, int cols, void* out,
                        cudaStream_t stream);
// inverse[copy] = row of the copy in the expert-ordered buffer, -1 when dropped.
// capacity < 0: padded layout; capacity >= 0: binned layout [E, capacity].
cudaError_t inverse_map(const int* indices, const int* bins, const int* padded_bins, int num_bins, int n,
                        int capacity, int* inverse_filled_minus_one, cudaStream_t stream);
cudaError_t combine_rows(DType type, const void* x, const int* inverse, const void* weights, int top_k,
                         int64_t tokens, int cols, void* out, cudaStream_t stream);
cudaError_t scatter_wgrad(DType type, const void* x, const void* grad, const int* inverse, int top_k,
                          int64_t copies, int cols, void* wgrad, cudaStream_t stream);

// ---- router.cu ----------------------------------------------------------------
constexpr int kRouterMaxExperts = 1024;
constexpr int kRouterMaxTopK = 8;
cudaError_t router_topk_fwd(DType type, const void* logits, int64_t tokens, int num_experts, int top_k,
                            float norm_p, void* scores, void* weights, int64_t* experts, cudaStream_t stream);
cudaError_t router_topk_bwd(DType type, const void* scores, const int64_t* experts, const void* dscores,
                            const void* dweights, int64_t tokens, int num_experts, int top_k, float norm_p,
                            void* dlogits, cudaStream_t stream);

// ---- optim.cu -----------------------------------------------------------------
struct AdamTensor {
  void* param;        // 16-bit (or fp32) shadow weights the model computes with
  const void* grad;
  float* master;      // fp32 weights
  float* exp_avg;
  float* exp_avg_sq;
  int64_t numel;
  float norm_weight;  // weight of this tensor in the squared gradient norm
  int pad_;
};
// `blocks[i] = {tensor index, chunk index}`; every CTA updates `chunk` elements.  `hyper` (nullable,
// device memory) = {lr, bias1, bias2}, read by the kernel in place of the arguments of those names.
cudaError_t adam_step(DType param_type, DType grad_type, const AdamTensor* tensors, const int2* blocks,
                      int num_blocks, int chunk, float lr, float beta1, float beta2, float eps, float weight_decay,
                      float bias1, float bias2, const float* grad_scale, const float* hyper, cudaStream_t stream);
cudaError_t grad_sqnorm(DType grad_type, const AdamTensor* tensors, const int2* blocks, int num_blocks, int chunk,
                        float* out_accum, cudaStream_t stream);
cudaError_t clip_coeff(const float* sqnorm, float max_norm, float extra_scale, float* out, cudaStream_t stream);

// ---- fused_ops.cu -------------------------------------------------------------
cudaError_t cross_entropy_fwd(DType type, const void* logits, const int64_t* targets, int64_t rows, int64_t vocab,
                              float* lse, float* loss, cudaStream_t stream);
// Overwrites `logits` with (softmax - onehot) * scale_ptr[0] * scale_mul.
// Loss per row into `loss`, and (softmax - onehot) * scale written over `logits`, in one launch.
cudaError_t cross_entropy_fused(DType type, void* logits, const int64_t* targets, float scale, int64_t rows,
                                int64_t vocab, float* loss, cudaStream_t stream);
cudaError_t cross_entropy_bwd(DType type, void* logits, const int64_t* targets, const float* lse,
                              const float* scale_ptr, float scale_mul, int64_t rows, int64_t vocab,
                              cudaStream_t stream);
int layernorm_grid(int64_t rows, int sms);   // CTAs (= rows of `partial`) the backward uses
// Optional fusions (rows short enough for the register kernels, see layernorm_fusable): forward
// normalises x + res (+ res_bias, a vector of `cols` values, when given) and writes the sum to
// sum_out; backward adds dres to dx.  `rms`: RMS norm
// (y = x * rsqrt(mean(x^2) + eps) * gamma; beta may be null, dbeta is then meaningless).
bool layernorm_fusable(DType type, int cols);
cudaError_t layernorm_fwd(DType type, const void* x, const void* gamma, const void* beta, int64_t rows, int cols,
                          float eps, void* y, float* mean, float* rstd, const void* res, const void* res_bias,
                          void* sum_out, bool rms, int sms, cudaStream_t stream);
cudaError_t layernorm_bwd(DType type, const void* dy, const void* x, const void* gamma, const float* mean,
                          const float* rstd, int64_t rows, int cols, void* dx, void* dgamma, void* dbeta,
                          float* partial, const void* dres, bool rms, int sms, cudaStream_t stream);

// Column sums of x[rows, cols] (cols a multiple of 16 bytes): `partial` holds slices x cols floats,
// slices = colsum_slices(...).
int colsum_slices(int64_t rows, int cols, int elem_size, int sms);
cudaError_t column_sum(DType type, const void* x, int64_t rows, int cols, void* out, float* partial, int slices,
                       cudaStream_t stream);

// ---- model_ops.cu -------------------------------------------------------------
constexpr int kLblMaxLayers = 64;
struct LblArgs {
  const void* scores[kLblMaxLayers];   // [tokens, experts] router scores of every layer
  const int* counts[kLblMaxLayers];    // [experts] tokens per expert of every layer
  void* dscores[kLblMaxLayers];        // backward: gradient of every layer's scores
};
int lbl_slices(int64_t tokens, int layers, int sms);
// loss = scale * sum over layers of <counts, column sums of scores>; `partial` holds layers x slices
// floats, `ticket` is a zeroed int.  Deterministic (fixed partition, fixed summation order).
cudaError_t lbl_forward(DType type, const LblArgs& args, int layers, int64_t tokens, int experts, float scale,
                        float* partial, int slices, int* ticket, float* loss, cudaStream_t stream);
// dscores[l][t, e] = gout[0] * scale * counts[l][e].
cudaError_t lbl_backward(DType type, const LblArgs& args, int layers, int64_t tokens, int experts, float scale,
                         const float* gout, int sms, cudaStream_t stream);
// Rotary embedding of x[batch, seq, heads, dim] (strides in elements, unit stride in dim) with
// cos / sin tables [seq, dim / 2]; `inverse` rotates the other way (the gradient).  out is contiguous.
cudaError_t rope(DType type, const void* x, int64_t stride_b, int64_t stride_s, int64_t stride_h, const float* cosv,
                 const float* sinv, int batch, int seq, int heads, int dim, bool inverse, void* out, int sms,
                 cudaStream_t stream);

// ---- ep_comm.cu ---------------------------------------------------------------
// Geometry of one expert-parallel workspace.  `peer_base[r]` is the address at which
// rank r's symmetric heap is mapped in this process (device array of `world` entries);
// offsets are byte offsets inside the heap, identical on every rank.
struct EpLayout {
  const uint64_t* peer_base;
  int world;
  int rank;
  int num_experts;
  int experts_per_rank;
  int capacity_rows;        // rows the receive buffers can hold (stores past it are skipped)
  int64_t off_counts;       // int32 [2][world][num_experts]
  int64_t off_count_flags;  // int32 [world]
  // Nullable: a counter in this GPU's memory whose value every kernel adds to the `seq` it was
  // launched with.  The host then keeps `seq` constant and bumps the counter with a stream-ordered
  // add, so a recorded launch (CUDA graph) takes a fresh sequence number at every replay.
  const int* seq_base;
};
constexpr int kEpErrCounts = 16, kEpErrOverflow = 17, kEpErrGemmWait = 18, kEpErrReturnWait = 19,
              kEpErrBufferBusy = 20;

// `counts_out` receives the [world][experts] matrix of routed copies, `kept_out` the copies that
// survive `expert_capacity` (rows kept per expert, counted over the sources in rank order; 0 = no
// limit, kept == counts), `recv_bins` the inclusive prefix sums of the kept rows of the local experts.
cudaError_t ep_exchange_counts(const int* tpe, const EpLayout& layout, int seq, int expert_capacity, int* counts_out,
                               int* kept_out, int* recv_bins, int* scratch_zero, int scratch_ints, int* status,
                               cudaStream_t stream);
// `data_base[r]` is the mapping of the heap that holds the row buffers (it may differ
// from the heap of the flags); `off_free < 0` skips the buffer-free handshake.  `counts` is the
// matrix of KEPT copies; a copy beyond its expert's kept count is not sent, and its row of
// `dropped_rows` (this rank's return buffer, sorted order; may be null) is cleared instead.
cudaError_t ep_push_rows(DType type, const void* x, const int* indices, const void* weights, const int* bins,
                         const int* counts, const EpLayout& layout, const uint64_t* data_base, int64_t off_recv,
                         int64_t off_flags, int64_t off_free, int seq, int top_k, int n, int cols, int* done,
                         int* status, void* dropped_rows, int sms, cudaStream_t stream);
// `counts` = kept copies (segment sizes here), `raw_counts` = routed copies (positions at the sources).
cudaError_t ep_return_rows(DType type, const void* y, const int* counts, const int* raw_counts,
                           const EpLayout& layout,
                           const uint64_t* data_base, int64_t off_ret, int64_t off_flags, int seq, int cols,
                           int rows_bound, int ret_rows, int* done, const int* status, int sms,
                           cudaStream_t stream);
cudaError_t ep_set_flag(int* flag, int value, const int* seq_base, cudaStream_t stream);
cudaError_t ep_wait_flags(const int* flags, int count, int seq, const int* seq_base, int* status, int code,
                          cudaStream_t stream);

// ---- dp_comm.cu ---------------------------------------------------------------
// Geometry of the data-parallel gradient heap: `peer_base[r]` is where rank r's symmetric heap is
// mapped in this process; the gradient buffer and the two flag arrays ([buckets][world] int32
// each) sit at the same byte offsets on every rank.
struct DpLayout {
  const uint64_t* peer_base;
  int world;
  int rank;
  int64_t off_grad;
  int64_t off_ready;
  int64_t off_done;
  const int* seq_base;   // nullable device counter added to `seq` (see EpLayout::seq_base)
};
constexpr int kDpErrReady = 32, kDpErrDone = 33;
// All-reduce (or, with `scatter_only`, reduce-scatter into this rank's slice) of elements
// [start, start + count) of the gradient buffer, times `scale`; `start` and `count` must be multiples
// of 16 bytes (for the reduce-scatter: `count` a multiple of world x 16 bytes, so that the slices are
// the callers' shards).  `ticket` is a zeroed device int owned by the bucket.
cudaError_t dp_allreduce(DType type, const DpLayout& layout, int64_t start, int64_t count, int bucket, int seq,
                         float scale, bool scatter_only, int* ticket, int* status, int ctas, cudaStream_t stream);

// ---- grouped GEMM ---------------------------------------------------------------
namespace gemm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kMaxGroups = 1024;

enum Layout : int { kNT = 0, kNN = 1, kTN = 2 };
enum Epilogue : int { kEpiNone = 0, kEpiAct = 1, kEpiDAct = 2, kEpiGlu = 3, kEpiDGlu = 4, kEpiAdd = 5, kEpiGluDual = 6 };
enum Act : int { kActIdentity = 0, kActGeluTanh = 1, kActSilu = 2, kActRelu = 3, kActGeluErf = 4 };

struct GemmParams {
  const int* bins;  // [num_groups] inclusive prefix sum of rows per group
  int num_groups;
  int rows_total;   // rows of a (and of c for NT / NN)
  int M;            // TN: rows of each output matrix
  int N;            // output columns per group
  int K;            // NT / NN: contraction length
  void* c;
  void* out2;
  void* out3;
  const void* aux1;
  const void* aux2;
  int epilogue;
  int act;
  float alpha;      // every accumulator is multiplied by this before the epilogue (1 = off)
  int* status;      // device word that receives a code when a wait is abandoned
  int zero_tail;    // NT / NN: write zeros to the rows of c past the last group
  // Optional arrival flags (expert-parallel receive buffer): before the first load of
  // a tile of group g the producer waits until wait_flags[s * wait_stride + g] >=
  // wait_seq for every s in [0, wait_count).  Null = no wait.
  const int* wait_flags;
  int wait_count;
  int wait_stride;
  int wait_seq;
  // Optional scatter of the main output (NN layout): instead of c[row], every output row is
  // stored into the return buffer of the rank it came from (expert-parallel combine fused into
  // the GEMM epilogue).  Rows of local expert j arrive grouped by source rank; the counts matrix
  // [world][experts] gives the segment sizes and the row offsets on the source side.  After the
  // last row for a source has been stored its flag is released.  Null scatter_base = off.
  const uint64_t* scatter_base;       // mapping of every rank's heap that holds the return buffer
  const uint64_t* scatter_flag_base;  // mapping of every rank's heap that holds the flags
  const int* scatter_counts;          // [world][experts] copies KEPT per (source, expert): segment sizes here
  const int* scatter_raw_counts;      // [world][experts] copies routed: positions in the sources' sorted order
  int* scatter_done;                  // [world] zeroed completion counters
  int64_t scatter_off;                // byte offset of the return buffer in its heap
  int64_t scatter_flag_off;           // byte offset of the int32 flag array [world] in its heap
  int scatter_world;
  int scatter_rank;
  int scatter_experts;                // global number of experts
  int scatter_seq;
  int scatter_rows;                   // rows of every rank's return buffer (stores past it are skipped)
  // Optional TMA stores of the outputs (single-CTA kernel): tensor maps of c / out2 / out3 viewed as
  // [rows, N] with 32 x 32 boxes and 64-byte swizzle.  Warps whose 32 rows of a tile all exist hand
  // their staged chunk to the TMA unit instead of storing it with the LSU.  0 = off.
  int store_tma;
  CUtensorMap out_map[3];
  // Second operand pair.
  //   dual_b (NT, block_n 256, epilogue kEpiGluDual): a tile covers 128 output columns and multiplies
  //   the same A tile with the matching 128 rows of b AND of b2 (one MMA with N = 256: accumulator
  //   columns [0, 128) = a b^T, [128, 256) = a b2^T).  Outputs: c = a b2^T, out2 = act(a b^T) * c,
  //   out3 = a b^T - the GLU forward in one launch.  Both B tensor maps then have 128-row boxes.
  //   k_concat (NN): the contraction runs over a x b and then over a2 x b2 into the same accumulator
  //   (c = a b + a2 b2: the GLU input gradient in one launch).
  int dual_b;
  int k_concat;
  int band_n;      // NT / NN: column tiles per band of the tile walk (0 = the kernel's default)
  CUtensorMap a2_map;
  CUtensorMap b2_map;
  // Nullable device counter added to wait_seq and scatter_seq (see EpLayout::seq_base).
  const int* seq_base;
  // TN only, nullable: one fp32 accumulator in device memory that receives the sum of squares of
  // everything the launch stores (the squared norm of a weight gradient, taken in the epilogue).
  float* sqnorm;
  // Diagnostics for roofline experiments (results are meaningless): bit 0 = the producer issues no
  // operand loads, bit 1 = the MMA warp issues no MMAs.  Set from MB200_GEMM_DIAG; 0 in normal use.
  int diag;
  // Role timers (builds with -DMB_GEMM_TIMING only): [grid][16] cycle counters, see the kernel.
  long long* timing;
};

// block_n is 64, 128 or 256.  The tensor maps describe a and b as row-major 16-bit
// matrices with 64-column boxes and 128-byte swizzle.
// `pair`: run the CTA-pair kernel (cta_group::2, 256-row tiles; block_n 256, even grid; for NT
// the B tensor map must then have 128-row boxes, NN and TN use the 64-row boxes of the single-CTA
// kernel).
cudaError_t launch(bool bf16, int layout, int block_n, const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                   const GemmParams& params, int grid, cudaStream_t stream, bool pair = false);

}  // namespace gemm

// ---- block-sparse products (bsmm.cu) ------------------------------------------------
namespace bsmm {

enum Mode : int { kSdd = 0, kDsd = 1, kDds = 2 };
constexpr int kBlock = 128;   // block size of the topology = edge of an output tile

// One launch computes every 128 x 128 output tile of one product over a BCSR topology with
// 128 x 128 blocks.  All index arrays are int32 device arrays.
struct BsmmParams {
  int mode;
  int num_tiles;
  int tiles_inner;             // dsd: column tiles per block row; dds: row tiles per block column
  int K;                       // sdd: dense contraction length
  const int* row_indices;      // sdd: block row of every stored block
  const int* column_indices;   // sdd: block column of every stored block
  // dsd / dds: per output block row (dsd) or block column (dds) j, the stored blocks
  // seg_offsets[j] .. seg_offsets[j + 1) to accumulate: seg_block[idx] is the position of the
  // block in the value array (null = idx itself), seg_k[idx] the 128-wide slice of the dense
  // operand it multiplies.
  const int* seg_offsets;
  const int* seg_block;
  const int* seg_k;
  void* out;                   // row-major 16-bit output
  int64_t out_ld;              // its row stride in elements
  int out_rows;
  int out_cols;
  int* status;
};

// The tensor maps describe the stored (row-major, 16-bit) operands with 64-column boxes and
// 128-byte swizzle: 128-row boxes for a K-major operand, 64-row boxes for an MN-major one.
cudaError_t launch(bool bf16, bool a_mn_major, bool b_mn_major, const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                   const BsmmParams& params, int grid, cudaStream_t stream);

}  // namespace bsmm
}  // namespace mb
