"""Gated-linear-unit experts: ``y = (act(x w1^T) * (x v1^T)) w2``.

Shapes and names follow the reference (megablocks/layers/glu.py:19-223): the
gate weight ``v1`` has the shape of ``w1`` and is initialised like it.  Both
dropless variants run the fused grouped kernels; unlike the reference the
block-sparse variant also supports ``memory_optimized_mlp``.
"""

import torch

from megablocks_b200.layers import mpu
from megablocks_b200.layers.arguments import Arguments
from megablocks_b200.layers.fused_mlp import expert_mlp
from megablocks_b200.layers.mlp import (SharedMLP, SparseMLP, _new_param, create_dmoe_expert_weights,
                                        resolve_dtensor)
from megablocks_b200.ops import gg as G
from megablocks_b200.ops import sparse


class SparseGLU(SparseMLP):

    def __init__(self, args: Arguments):
        super().__init__(args)
        self.v1 = _new_param(args, self._num_rows_per_rank, args.hidden_size)
        with torch.no_grad():
            self.v1.copy_(
                create_dmoe_expert_weights(args, args.moe_num_experts, args.ffn_hidden_size, args.hidden_size,
                                           args.init_method))
        mpu.set_expert_model_parallel_attributes(self.v1, self._should_set_parallelism_attribute)

    def _glu_weights(self):
        w1, w2 = self._weights()
        v1 = resolve_dtensor(self.scale_grad(self.v1))
        return w1, v1, w2

    def _raw_glu_weights(self):
        """Weights without the gradient-scaling node (pair with ``wgrad_scale()``)."""
        w1, w2 = self._raw_weights()
        return w1, resolve_dtensor(self.v1), w2

    def forward(self, x: torch.Tensor, topo) -> torch.Tensor:
        padded_bins = getattr(topo, 'padded_bins', None)
        if padded_bins is not None:
            w1, v1, w2 = self._raw_glu_weights()
            return expert_mlp(x, self._grouped_view(w1), self._grouped_view(w2), padded_bins,
                              self.args.activation_fn, self.args.memory_optimized_mlp, v1=self._grouped_view(v1),
                              wgrad_scale=self.wgrad_scale())
        w1, v1, w2 = self._glu_weights()
        gate = sparse.sdd(x, w1.t(), topo)
        up = sparse.sdd(x, v1.t(), topo)
        hidden = sparse.mul(sparse.with_data(gate, self.args.activation_fn(gate.data)), up)
        return sparse.dsd(hidden, w2)


class GroupedGLU(SparseGLU):

    def forward(self, x: torch.Tensor, tokens_per_expert: torch.Tensor, bins=None) -> torch.Tensor:
        w1, v1, w2 = self._raw_glu_weights()
        if bins is None:
            bins = torch.cumsum(tokens_per_expert, 0, dtype=torch.int32)
        return expert_mlp(x, self._grouped_view(w1), self._grouped_view(w2), bins, self.args.activation_fn,
                          self.args.memory_optimized_mlp, v1=self._grouped_view(v1), wgrad_scale=self.wgrad_scale())


def memory_optimized_grouped_glu(x, w1, v1, w2, batch_sizes, activation_fn):
    """Functional grouped GLU (weights ``[E, f, h]``) with activation recompute."""
    bins = G.bins_from_batch_sizes(batch_sizes, x.device)
    return expert_mlp(x, w1, w2, bins, activation_fn, True, v1=v1)


class SharedGLU(SharedMLP):
    """Shared expert with a gate projection: ``down(act(gate(x)) * up(x))``."""

    def __init__(self, args: Arguments):
        super().__init__(args)
        self.gate_proj = args.fc_cls(args.hidden_size, args.shared_expert_hidden_size, **self.fc_kwargs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.act(self.gate_proj(x)) * self.up_proj(x))
