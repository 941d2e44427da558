"""Dropless MoE: every routed copy is computed, no capacity limit.

Reference behaviour: megablocks/layers/dmoe.py:18-326.  Two layouts:

* ``mlp_impl='sparse'``: copies are gathered into a buffer where each expert's
  rows are padded to a multiple of 128; the expert computation is the
  block-diagonal block-sparse product ``dsd(act(sdd(x, w1^T)), w2)``.
* ``mlp_impl='grouped'``: copies are gathered contiguously and the experts run
  as a grouped GEMM over ragged row groups.

Both end up on the same tcgen05 grouped kernel.  The padded buffer is sized by
a static upper bound (``copies + E * 127`` rounded up to 128) instead of the
data-dependent exact size, so the forward pass never waits for the device;
row-blocks past the last expert are zero and cost no FLOPs.
"""

import torch

from megablocks_b200 import ops
from megablocks_b200.layers import common, dmlp_registry, moe, mpu
from megablocks_b200.layers.arguments import Arguments
from megablocks_b200.ops import sparse


def promote_scalar(x: torch.Tensor) -> torch.Tensor:
    return x.view(1) if x.dim() == 0 else x


class ParallelDroplessMLP(moe.ParallelMLP):

    def __init__(self, args: Arguments):
        self.blocking = 128
        super().__init__(args)
        self.hidden_size = args.hidden_size
        self.ffn_hidden_size = mpu.features_per_rank(args)
        max_column_index = (self.ffn_hidden_size * self.num_experts) // self.blocking
        self.transpose_sort_end_bit = max(int(max_column_index - 1).bit_length(), 1)
        if args.moe_expert_model_parallelism:
            self.forward_fn = self.parallel_forward_once

    def _build_experts(self, args: Arguments) -> torch.nn.Module:
        return dmlp_registry.get(args)

    # -- topology -------------------------------------------------------------
    def sparse_transpose(self, size, row_indices, column_indices, offsets):
        """Transpose metadata ``(column_indices_t, offsets_t, block_offsets_t)`` of a BCSR topology."""
        return sparse._transpose_metadata(size, self.blocking, row_indices, column_indices)

    def padded_rows_bound(self, copies: int) -> int:
        """Static upper bound of ``padded_bins[-1]`` for ``copies`` routed rows."""
        experts = mpu.experts_per_rank(self.args) if self.args.moe_expert_model_parallelism else self.num_experts
        worst = copies + experts * (self.blocking - 1)
        return ((worst + self.blocking - 1) // self.blocking) * self.blocking

    def topology(self, x: torch.Tensor, padded_bins: torch.Tensor) -> sparse.Matrix:
        """Block-diagonal topology of the hidden activation ``[padded_rows, E_local * ffn]``.

        The block values are a zero-storage placeholder (shape only), as in the
        reference where the topology is a pure index carrier.
        """
        padded_tokens = x.shape[0]
        if padded_tokens % self.blocking:
            raise ValueError('the padded token count must be a multiple of the block size')
        if self.ffn_hidden_size % self.blocking:
            raise ValueError(f'The ffn_hidden_size {self.ffn_hidden_size} must be divisible by '
                             f'the block size {self.blocking}. Please update your configuration.')
        block_rows = padded_tokens // self.blocking
        blocks_per_row = self.ffn_hidden_size // self.blocking
        offsets = torch.arange(0, block_rows * blocks_per_row + 1, blocks_per_row, dtype=torch.int32,
                               device=x.device)
        column_indices = ops.topology(padded_bins, self.blocking, block_rows, blocks_per_row)
        data = torch.empty(column_indices.numel(), self.blocking, self.blocking, dtype=common.dtype(self.args),
                           device='meta')
        shape = (padded_tokens, self.ffn_hidden_size * mpu.experts_per_rank(self.args))
        row_indices = torch.arange(block_rows, dtype=torch.int16, device=x.device).repeat_interleave(blocks_per_row)
        # Row-block r holds `blocks_per_row` consecutive column-blocks, so the
        # transpose is closed-form: column-block c of expert e lists that
        # expert's row-blocks in order.  Build it lazily only if asked for.
        topo = _LazyTopology(shape, data, row_indices, column_indices, offsets)
        topo.padded_bins = padded_bins
        return topo

    def indices_and_padded_bins(self, top_experts: torch.Tensor):
        indices, bin_ids, bins, padded_bins, tokens_per_expert = ops.route_plan(top_experts, self.num_experts,
                                                                                self.blocking)
        return indices, bin_ids, bins, padded_bins, tokens_per_expert

    # -- block-sparse layout ---------------------------------------------------
    def sparse_forward_once(self, x, expert_weights, top_experts):
        expert_weights = expert_weights.flatten()
        top_experts = top_experts.flatten()
        with torch.no_grad():
            indices, bin_ids, bins, padded_bins, tokens_per_expert = self.indices_and_padded_bins(top_experts)
        x = x.reshape(-1, x.shape[-1])
        x = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, self.top_k,
                              num_rows=self.padded_rows_bound(indices.numel()))
        with torch.no_grad():
            topo = self.topology(x, padded_bins)
        x = self.mlp(x, topo)
        x = ops.padded_scatter(x, indices, bin_ids, expert_weights, bins, padded_bins, self.top_k)
        return x, tokens_per_expert

    def sparse_permute_and_compute(self, x, tokens_per_expert, indices, bin_ids, expert_weights, bins,
                                   expert_capactiy, top_k):
        """Expert-parallel inner step on the padded layout (``tokens_per_expert`` is device-side)."""
        with torch.no_grad():
            padded = ops.round_up(tokens_per_expert, self.blocking)
            padded_bins = promote_scalar(ops.inclusive_cumsum(padded, 0))
        x = x.reshape(-1, x.shape[-1])
        x = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k,
                              num_rows=self.padded_rows_bound(indices.numel()))
        with torch.no_grad():
            topo = self.topology(x, padded_bins)
        x = self.mlp(x, topo)
        return ops.padded_scatter(x, indices, bin_ids, expert_weights, bins, padded_bins, top_k)

    # -- grouped layout --------------------------------------------------------
    def grouped_forward_once(self, x, expert_weights, top_experts):
        expert_weights = expert_weights.flatten()
        top_experts = top_experts.flatten()
        with torch.no_grad():
            indices, bin_ids, bins, tokens_per_expert = self.indices_and_bins(top_experts)
        out = self.grouped_permute_and_compute(x, tokens_per_expert, indices, bin_ids, expert_weights, bins, -1,
                                               self.top_k)
        return out, tokens_per_expert

    def grouped_permute_and_compute(self, x, tokens_per_expert, indices, bin_ids, expert_weights, bins,
                                    expert_capactiy, top_k):
        x = x.reshape(-1, x.shape[-1])
        x = ops.gather(x, indices, bin_ids, bins, top_k)
        x = self.mlp(x, tokens_per_expert, bins=bins)      # bins = prefix sum of tokens_per_expert
        return ops.scatter(x, indices, bin_ids, expert_weights, bins, top_k)

    # -- expert parallel over peer memory ----------------------------------------
    def parallel_forward_once(self, x, expert_weights, top_experts):
        if not self._use_fused_ep(x):
            return super().parallel_forward_once(x, expert_weights, top_experts)
        mlp = self.mlp
        # Unscaled weights: the 1 / world factor of their gradients is applied inside the wgrad GEMMs.
        w1, w2 = mlp._raw_weights()
        v1 = None
        if self.args.mlp_type == 'glu':
            w1, v1, w2 = mlp._raw_glu_weights()
            v1 = mlp._grouped_view(v1)
        return self.fused_parallel_forward_once(x, expert_weights, top_experts, mlp._grouped_view(w1),
                                                mlp._grouped_view(w2), v1, w1_kn=False, expert_capacity=0)

    # -- dispatch --------------------------------------------------------------
    def forward_once(self, x, expert_weights, top_experts):
        if self.args.mlp_impl == 'sparse':
            return self.sparse_forward_once(x, expert_weights, top_experts)
        return self.grouped_forward_once(x, expert_weights, top_experts)

    def permute_and_compute(self, x, tokens_per_expert, indices, bin_ids, expert_weights, bins, expert_capactiy,
                            top_k):
        if self.args.mlp_impl == 'sparse':
            return self.sparse_permute_and_compute(x, tokens_per_expert, indices, bin_ids, expert_weights, bins,
                                                   expert_capactiy, top_k)
        return self.grouped_permute_and_compute(x, tokens_per_expert, indices, bin_ids, expert_weights, bins,
                                                expert_capactiy, top_k)


class _LazyTopology(sparse.Matrix):
    """Topology whose transpose metadata is materialised on first use."""

    def __init__(self, size, data, row_indices, column_indices, offsets):
        self._size = tuple(int(s) for s in size)
        self.data = data
        self.row_indices = row_indices
        self.column_indices = column_indices
        self.offsets = offsets
        self._transposed = False
        self.padded_bins = None
        self._t_meta = None

    def _meta(self):
        if self._t_meta is None:
            self._t_meta = sparse._transpose_metadata(self._size, int(self.data.shape[1]), self.row_indices,
                                                      self.column_indices)
        return self._t_meta

    @property
    def column_indices_t(self):
        return self._meta()[0]

    @property
    def offsets_t(self):
        return self._meta()[1]

    @property
    def block_offsets_t(self):
        return self._meta()[2]


class dMoE(moe.MoE):

    def _init_experts_mlp(self, args: Arguments) -> ParallelDroplessMLP:
        return ParallelDroplessMLP(args)
