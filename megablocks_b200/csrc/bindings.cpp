// Python bindings of the sm_100a extension (module megablocks_b200._C).
#include <torch/extension.h>

#include <vector>

namespace mb {

// torch_glue.cpp: metadata
std::vector<at::Tensor> sort_pairs(const at::Tensor& x, int64_t end_bit);
std::vector<at::Tensor> route_plan(const at::Tensor& top_experts, int64_t num_experts, int64_t block);
at::Tensor histogram_op(const at::Tensor& x, int64_t num_bins);
at::Tensor cumsum_op(const at::Tensor& x, bool exclusive);
at::Tensor topology_op(const at::Tensor& padded_bins, int64_t block_size, int64_t rows, int64_t cols);
at::Tensor replicate_forward(const at::Tensor& x, const at::Tensor& bins, int64_t num_outputs);
at::Tensor replicate_backward(const at::Tensor& grad, const at::Tensor& bins);

// torch_glue.cpp: permutation
at::Tensor gather_rows_op(const at::Tensor& x, const at::Tensor& indices, const at::Tensor& bin_ids,
                       const c10::optional<at::Tensor>& weights, const at::Tensor& bins,
                       const at::Tensor& padded_bins, int64_t top_k, int64_t out_rows);
at::Tensor scatter_rows_op(const at::Tensor& x, const at::Tensor& indices, const at::Tensor& bin_ids,
                        const c10::optional<at::Tensor>& weights, const at::Tensor& bins,
                        const at::Tensor& padded_bins, int64_t top_k, int64_t tokens);
at::Tensor scatter_wgrad_op(const at::Tensor& x, const at::Tensor& grad, const at::Tensor& indices,
                         const at::Tensor& bin_ids, const at::Tensor& bins, const at::Tensor& padded_bins,
                         int64_t top_k);
at::Tensor binned_gather_rows(const at::Tensor& x, const at::Tensor& indices,
                              const c10::optional<at::Tensor>& weights, const at::Tensor& bins, int64_t capacity,
                              int64_t top_k);
at::Tensor binned_scatter_rows(const at::Tensor& x, const at::Tensor& indices,
                               const c10::optional<at::Tensor>& weights, const at::Tensor& bins, int64_t top_k,
                               int64_t tokens);
at::Tensor binned_scatter_wgrad(const at::Tensor& x, const at::Tensor& grad, const at::Tensor& indices,
                                const at::Tensor& bins, int64_t top_k);

// torch_glue.cpp: router
std::vector<at::Tensor> router_topk_forward(const at::Tensor& logits, int64_t top_k, double norm_p);
at::Tensor router_topk_backward(const at::Tensor& scores, const at::Tensor& weights, const at::Tensor& experts,
                                const at::Tensor& dscores, const at::Tensor& dweights, double norm_p);

// torch_glue.cpp: grouped GEMM
bool grouped_gemm_supported(const at::Tensor& a, const at::Tensor& b, bool trans_a, bool trans_b,
                            int64_t num_groups);
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
                                     const c10::optional<at::Tensor>& seq_base);
int64_t read_status(bool clear);
int64_t launch_count();
void count_launches(int64_t n);
at::Tensor gemm_role_timers(const at::Tensor& like);
at::Tensor bsmm_op(int64_t mode, const at::Tensor& a, bool a_mn, const at::Tensor& b, bool b_mn,
                   const at::Tensor& idx0, const c10::optional<at::Tensor>& idx1,
                   const c10::optional<at::Tensor>& idx2, int64_t out_rows, int64_t out_cols);

// torch_glue.cpp: symmetric heap and expert-parallel exchange
std::vector<at::Tensor> symm_alloc(int64_t nbytes);
int64_t symm_open(const at::Tensor& handle);
void symm_close(int64_t ptr);
void ep_exchange_counts_op(const at::Tensor& tpe, const at::Tensor& peer_base, int64_t world, int64_t rank,
                           int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows, int64_t off_counts,
                           int64_t off_count_flags, int64_t seq, int64_t expert_capacity, at::Tensor counts_out,
                           at::Tensor kept_out, at::Tensor recv_bins, at::Tensor scratch,
                           const c10::optional<at::Tensor>& seq_base);
void ep_push_rows_op(const at::Tensor& x, const at::Tensor& indices, const c10::optional<at::Tensor>& weights,
                     const at::Tensor& bins, const at::Tensor& counts, const at::Tensor& peer_base, int64_t world,
                     int64_t rank, int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows,
                     int64_t off_counts, int64_t off_count_flags, const at::Tensor& data_base, int64_t off_recv,
                     int64_t off_flags, int64_t off_free, int64_t seq, int64_t top_k, at::Tensor done,
                     const c10::optional<at::Tensor>& dropped_rows, const c10::optional<at::Tensor>& seq_base);
void ep_return_rows_op(const at::Tensor& y, const at::Tensor& counts, const at::Tensor& raw_counts,
                       const at::Tensor& peer_base, int64_t world,
                       int64_t rank, int64_t num_experts, int64_t experts_per_rank, int64_t capacity_rows,
                       int64_t off_counts, int64_t off_count_flags, const at::Tensor& data_base, int64_t off_ret,
                       int64_t off_flags, int64_t seq, int64_t ret_rows, at::Tensor done,
                       const c10::optional<at::Tensor>& seq_base);
void ep_set_flag_op(at::Tensor flag, int64_t value, const c10::optional<at::Tensor>& seq_base);
void dp_allreduce_op(const at::Tensor& like, const at::Tensor& peer_base, int64_t world, int64_t rank,
                     int64_t off_grad, int64_t off_ready, int64_t off_done, int64_t start, int64_t count,
                     int64_t bucket, int64_t seq, double scale, bool scatter_only, at::Tensor ticket, int64_t ctas,
                     const c10::optional<at::Tensor>& seq_base);
void ep_wait_flags_op(const at::Tensor& flags, int64_t count, int64_t seq, int64_t code,
                      const c10::optional<at::Tensor>& seq_base);

// torch_glue.cpp: fused row-wise ops
std::vector<at::Tensor> cross_entropy_forward(const at::Tensor& logits, const at::Tensor& targets);
at::Tensor cross_entropy_fused_(at::Tensor logits, const at::Tensor& targets, double scale);
void cross_entropy_backward_(at::Tensor logits, const at::Tensor& targets, const at::Tensor& lse,
                             const c10::optional<at::Tensor>& scale, double scale_mul);
std::vector<at::Tensor> layernorm_forward(const at::Tensor& x, const at::Tensor& gamma,
                                          const c10::optional<at::Tensor>& beta, double eps,
                                          const c10::optional<at::Tensor>& res,
                                          const c10::optional<at::Tensor>& res_bias);
std::vector<at::Tensor> layernorm_backward(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gamma,
                                           const at::Tensor& mean, const at::Tensor& rstd,
                                           const c10::optional<at::Tensor>& dres, bool rms);
bool layernorm_can_fuse(const at::Tensor& x);
at::Tensor lbl_forward_op(const std::vector<at::Tensor>& scores, const std::vector<at::Tensor>& counts, double scale);
std::vector<at::Tensor> lbl_backward_op(const std::vector<at::Tensor>& scores, const std::vector<at::Tensor>& counts,
                                        double scale, const at::Tensor& gout);
at::Tensor rope_op(const at::Tensor& x, const at::Tensor& cosv, const at::Tensor& sinv, bool inverse);
at::Tensor column_sum_op(const at::Tensor& x);

// torch_glue.cpp: optimizer
int64_t adam_record_size();
void adam_step_op(const at::Tensor& table, const at::Tensor& blocks, int64_t chunk, int64_t param_code,
                  int64_t grad_code, double lr, double beta1, double beta2, double eps, double weight_decay,
                  double bias1, double bias2, const c10::optional<at::Tensor>& grad_scale,
                  const c10::optional<at::Tensor>& hyper);
void grad_sqnorm_op(const at::Tensor& table, const at::Tensor& blocks, int64_t chunk, int64_t grad_code,
                    at::Tensor out_accum);
void clip_coeff_op(const at::Tensor& sqnorm, double max_norm, double extra_scale, at::Tensor out);

}  // namespace mb

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "megablocks_b200 sm_100a kernels";
  m.def("sort_pairs", &mb::sort_pairs);
  m.def("route_plan", &mb::route_plan);
  m.def("histogram", &mb::histogram_op);
  m.def("cumsum", &mb::cumsum_op);
  m.def("topology", &mb::topology_op);
  m.def("replicate_forward", &mb::replicate_forward);
  m.def("replicate_backward", &mb::replicate_backward);
  m.def("gather_rows", &mb::gather_rows_op);
  m.def("scatter_rows", &mb::scatter_rows_op);
  m.def("scatter_wgrad", &mb::scatter_wgrad_op);
  m.def("binned_gather_rows", &mb::binned_gather_rows);
  m.def("binned_scatter_rows", &mb::binned_scatter_rows);
  m.def("binned_scatter_wgrad", &mb::binned_scatter_wgrad);
  m.def("router_topk_forward", &mb::router_topk_forward);
  m.def("router_topk_backward", &mb::router_topk_backward);
  m.def("grouped_gemm_supported", &mb::grouped_gemm_supported);
  m.def("grouped_gemm", &mb::grouped_gemm);
  m.def("read_status", &mb::read_status);
  m.def("launch_count", &mb::launch_count);
  m.def("count_launches", &mb::count_launches);
  m.def("gemm_role_timers", &mb::gemm_role_timers,
        "Per-CTA cycle counters of the grouped GEMM roles (builds with -DMB_GEMM_TIMING)");
  m.def("cross_entropy_forward", &mb::cross_entropy_forward);
  m.def("cross_entropy_backward_", &mb::cross_entropy_backward_);
  m.def("cross_entropy_fused_", &mb::cross_entropy_fused_,
        "Per-row loss; the logits are overwritten with (softmax - onehot) * scale in the same launch");
  m.def("layernorm_forward", &mb::layernorm_forward);
  m.def("layernorm_backward", &mb::layernorm_backward);
  m.def("layernorm_can_fuse", &mb::layernorm_can_fuse);
  m.def("lbl_forward", &mb::lbl_forward_op, "Load-balancing loss of all layers in one reduction kernel");
  m.def("lbl_backward", &mb::lbl_backward_op);
  m.def("rope", &mb::rope_op, "Rotary position embedding of [batch, seq, heads, dim]");
  m.def("column_sum", &mb::column_sum_op, "Sum over rows of x[rows, cols] (bias gradient)");
  m.def("symm_alloc", &mb::symm_alloc);
  m.def("symm_open", &mb::symm_open);
  m.def("symm_close", &mb::symm_close);
  m.def("bsmm", &mb::bsmm_op,
        "Block-sparse sdd (0) / dsd (1) / dds (2) over 128 x 128 blocks on tcgen05 tensor cores");
  m.def("ep_exchange_counts", &mb::ep_exchange_counts_op);
  m.def("ep_push_rows", &mb::ep_push_rows_op);
  m.def("ep_return_rows", &mb::ep_return_rows_op);
  m.def("ep_wait_flags", &mb::ep_wait_flags_op);
  m.def("ep_set_flag", &mb::ep_set_flag_op);
  m.def("dp_allreduce", &mb::dp_allreduce_op,
        "Gradient bucket all-reduce / reduce-scatter over peer memory (one kernel, bounded waits)");
  m.def("adam_record_size", &mb::adam_record_size);
  m.def("adam_step", &mb::adam_step_op);
  m.def("grad_sqnorm", &mb::grad_sqnorm_op);
  m.def("clip_coeff", &mb::clip_coeff_op);
}
