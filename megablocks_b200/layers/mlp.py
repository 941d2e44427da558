"""Expert MLPs: batched (token-dropping MoE), block-sparse, grouped and shared.

Parameter shapes, names and initialisation follow the reference so state dicts
are interchangeable (megablocks/layers/mlp.py:43-167, 308-394, 499-574):

* ``MLP``        ``w1 [E_local, hidden, ffn_local]``, ``w2 [E_local, ffn_local, hidden]``;
* ``SparseMLP`` / ``GroupedMLP``  ``w1, w2 [E_local * ffn_local, hidden]``.

Weights are drawn as one full ``[E, ffn, hidden]`` tensor and then sliced to
this rank's experts and ffn rows, so a given seed yields the same model at any
expert-parallel degree.  Under expert parallelism the expert weights carry
``expert_model_parallel = True`` and their gradients are pre-scaled by
``1 / ep_world`` so that a trainer averaging over all data-parallel ranks ends
up with the right magnitude.

All expert products run on the grouped tcgen05 kernel; there is no copy of row
counts to the host anywhere in the forward or backward pass.
"""

from typing import Any, Optional

import torch

from megablocks_b200.layers import common, mpu
from megablocks_b200.layers.arguments import Arguments, InitFn
from megablocks_b200.layers.fused_mlp import expert_mlp
from megablocks_b200.ops import gg as G
from megablocks_b200.ops import sparse


class ScaleGradient(torch.autograd.Function):
    """Identity in forward; multiplies the gradient by a constant in backward."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, scale: float):
        ctx.scale = scale
        return x

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor):
        return grad * ctx.scale, None


scale_gradient = ScaleGradient.apply


def resolve_dtensor(weight: torch.Tensor) -> torch.Tensor:
    """Local shard of a DTensor parameter; any other tensor is returned as is."""
    try:
        from torch.distributed.tensor import DTensor
    except ImportError:  # pragma: no cover
        return weight
    if isinstance(weight, DTensor):
        return weight.to_local()
    return weight


def _rank_slice(args: Arguments, num_experts: int, ffn_hidden_size: int):
    """(expert range, ffn-row range) owned by this expert-parallel rank."""
    esd = mpu.expert_sharding_degree(args)
    hsd = mpu.hidden_sharding_degree(args)
    rank = mpu.get_expert_parallel_rank(args)
    per_rank = num_experts // esd
    rows = ffn_hidden_size // hsd
    e0 = (rank % esd) * per_rank
    r0 = (rank // esd) * rows
    return slice(e0, e0 + per_rank), slice(r0, r0 + rows)


def create_moe_expert_weights(args: Arguments, num_experts: int, ffn_hidden_size: int, hidden_size: int,
                              init_method: InitFn) -> torch.Tensor:
    """``[E_local, ffn_local, hidden]`` slice of a freshly initialised full weight tensor."""
    full = torch.empty(num_experts, ffn_hidden_size, hidden_size, device=args.device, dtype=common.dtype(args))
    init_method(full)
    if not args.moe_expert_model_parallelism:
        return full
    experts, rows = _rank_slice(args, num_experts, ffn_hidden_size)
    with torch.no_grad():
        return full[experts, rows]


def create_dmoe_expert_weights(args: Arguments, num_experts: int, ffn_hidden_size: int, hidden_size: int,
                               init_method: InitFn) -> torch.Tensor:
    """The same slice flattened to ``[E_local * ffn_local, hidden]``."""
    weights = create_moe_expert_weights(args, num_experts, ffn_hidden_size, hidden_size, init_method)
    return weights.reshape(-1, hidden_size)


def _new_param(args: Arguments, *shape) -> torch.nn.Parameter:
    return torch.nn.Parameter(torch.empty(*shape, device=args.device, dtype=common.dtype(args)))


class _ExpertWeights(torch.nn.Module):
    """Shared plumbing: EP tagging and gradient pre-scaling of expert weights."""

    def _finish_init(self, args: Arguments, *params: torch.nn.Parameter) -> None:
        self._should_set_parallelism_attribute = args.moe_expert_model_parallelism
        for p in params:
            mpu.set_expert_model_parallel_attributes(p, self._should_set_parallelism_attribute)
        self.gradient_scale = None
        if args.moe_expert_model_parallelism:
            self.gradient_scale = 1 / mpu.get_expert_parallel_world_size(args)

    def scale_grad(self, w: torch.Tensor) -> torch.Tensor:
        if self.gradient_scale is None:
            return w
        return scale_gradient(w, self.gradient_scale)

    def wgrad_scale(self) -> float:
        """Factor for the fused expert MLP, which scales weight gradients inside their GEMMs."""
        return 1.0 if self.gradient_scale is None else float(self.gradient_scale)


class MLP(_ExpertWeights):
    """Experts applied to a dense ``[E_local, capacity, hidden]`` batch."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.args = args
        experts = mpu.experts_per_rank(args)
        features = mpu.features_per_rank(args)
        self.w1 = _new_param(args, experts, args.hidden_size, features)
        self.w2 = _new_param(args, experts, features, args.hidden_size)
        # Parameters are allocated before the full-size initialisation tensors
        # so the allocator cannot hand the same block to both.
        with torch.no_grad():
            w1 = create_moe_expert_weights(args, args.moe_num_experts, args.ffn_hidden_size, args.hidden_size,
                                           args.init_method)
            self.w1.copy_(w1.transpose(1, 2).contiguous())
            self.w2.copy_(
                create_moe_expert_weights(args, args.moe_num_experts, args.ffn_hidden_size, args.hidden_size,
                                          args.output_layer_init_method))
        self._finish_init(args, self.w1, self.w2)
        self._bins_cache = {}

    def _uniform_bins(self, experts: int, capacity: int, device) -> torch.Tensor:
        key = (experts, capacity, str(device))
        if key not in self._bins_cache:
            self._bins_cache[key] = (torch.arange(1, experts + 1, dtype=torch.int32, device=device) * capacity)
        return self._bins_cache[key]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w1 = resolve_dtensor(self.scale_grad(self.w1))
        w2 = resolve_dtensor(self.scale_grad(self.w2))
        experts, capacity, hidden = x.shape
        if capacity == 0:
            return x.new_zeros(experts, 0, w2.shape[-1])
        bins = self._uniform_bins(experts, capacity, x.device)
        z = G.gmm_bins(x.reshape(experts * capacity, hidden), w1, bins)
        y = G.gmm_bins(self.args.activation_fn(z), w2, bins)
        return y.view(experts, capacity, -1)


class SparseMLP(_ExpertWeights):
    """dMoE experts on the 128-row block-padded layout (block-sparse formulation)."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.args = args
        self._num_rows_per_rank = mpu.experts_per_rank(args) * mpu.features_per_rank(args)
        self.w1 = _new_param(args, self._num_rows_per_rank, args.hidden_size)
        self.w2 = _new_param(args, self._num_rows_per_rank, args.hidden_size)
        with torch.no_grad():
            self.w1.copy_(
                create_dmoe_expert_weights(args, args.moe_num_experts, args.ffn_hidden_size, args.hidden_size,
                                           args.init_method))
            self.w2.copy_(
                create_dmoe_expert_weights(args, args.moe_num_experts, args.ffn_hidden_size, args.hidden_size,
                                           args.output_layer_init_method))
        self._finish_init(args, self.w1, self.w2)

    def _weights(self):
        w1 = resolve_dtensor(self.scale_grad(self.w1))
        w2 = resolve_dtensor(self.scale_grad(self.w2))
        return w1, w2

    def _raw_weights(self):
        """Weights without the gradient-scaling node (pair with :meth:`wgrad_scale`)."""
        return resolve_dtensor(self.w1), resolve_dtensor(self.w2)

    def _grouped_view(self, w: torch.Tensor) -> torch.Tensor:
        return w.view(mpu.experts_per_rank(self.args), -1, self.args.hidden_size)

    def forward(self, x: torch.Tensor, topo) -> torch.Tensor:
        """``topo`` is a block-sparse :class:`~megablocks_b200.ops.sparse.Matrix`.

        Topologies built by the dMoE layer are block-diagonal and carry
        ``padded_bins``; they go straight to the grouped kernel.  Any other
        topology runs the general sdd / dsd products.
        """
        padded_bins = getattr(topo, 'padded_bins', None)
        if padded_bins is not None:
            w1, w2 = self._raw_weights()
            return expert_mlp(x, self._grouped_view(w1), self._grouped_view(w2), padded_bins,
                              self.args.activation_fn, self.args.memory_optimized_mlp,
                              wgrad_scale=self.wgrad_scale())
        w1, w2 = self._weights()
        hidden = sparse.sdd(x, w1.t(), topo)
        hidden = sparse.with_data(hidden, self.args.activation_fn(hidden.data))
        return sparse.dsd(hidden, w2)


class GroupedMLP(SparseMLP):
    """dMoE experts on the unpadded expert-ordered layout."""

    def forward(self, x: torch.Tensor, tokens_per_expert: torch.Tensor, bins=None) -> torch.Tensor:
        """``tokens_per_expert`` is the per-expert row count (device tensor; no host copy is made);
        ``bins`` its inclusive prefix sum when the caller already has it."""
        w1, w2 = self._raw_weights()
        if bins is None:
            bins = torch.cumsum(tokens_per_expert, 0, dtype=torch.int32)
        return expert_mlp(x, self._grouped_view(w1), self._grouped_view(w2), bins, self.args.activation_fn,
                          self.args.memory_optimized_mlp, wgrad_scale=self.wgrad_scale())


def memory_optimized_mlp(x, w1, w2, topo, activation_fn):
    """Functional block-sparse MLP that keeps only ``x`` and the pre-activation.

    ``w1``/``w2`` are ``[E*f, h]``; ``topo`` must be a dMoE topology (it carries
    ``padded_bins``).
    """
    experts = topo.padded_bins.numel()
    return expert_mlp(x, w1.view(experts, -1, w1.shape[-1]), w2.view(experts, -1, w2.shape[-1]), topo.padded_bins,
                      activation_fn, True)


def memory_optimized_grouped_mlp(x, w1, w2, batch_sizes, activation_fn):
    """Functional grouped MLP (``w1``/``w2`` are ``[E, f, h]``) with activation recompute."""
    bins = G.bins_from_batch_sizes(batch_sizes, x.device)
    return expert_mlp(x, w1, w2, bins, activation_fn, True)


class SharedMLP(torch.nn.Module):
    """Dense expert applied to every token, built from ``args.fc_cls`` layers."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.args = args
        self.fc_kwargs = {'bias': args.bias, 'device': args.device}
        self.fc_kwargs.update(args.fc_kwargs)
        self.up_proj = args.fc_cls(args.hidden_size, args.shared_expert_hidden_size, **self.fc_kwargs)
        self.act = args.activation_fn
        self.down_proj = args.fc_cls(args.shared_expert_hidden_size, args.hidden_size, **self.fc_kwargs)
        self.down_proj._is_residual = True  # read by llm-foundry style initialisers

    def add_experts_sharedexpert(self, shared_expert_out: torch.Tensor, expert_out: torch.Tensor) -> torch.Tensor:
        """Combine with the routed experts: plain add, or a (1, k)/(k+1) weighted sum."""
        if self.args.shared_expert_weighted_sum:
            parts = self.args.moe_top_k + 1
            return (shared_expert_out / parts).add(expert_out, alpha=self.args.moe_top_k / parts)
        return shared_expert_out + expert_out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.act(self.up_proj(x)))
