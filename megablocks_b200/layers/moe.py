"""Token-dropping MoE, the expert-parallel engine and the load-balancing loss.

Behaviour follows the reference layer (megablocks/layers/moe.py:14-475):

* ``ParallelMLP`` routes copies to experts, runs them and un-routes the result,
  on one device (``forward_once``) or across an expert-parallel group
  (``parallel_forward_once``);
* ``MoE`` = router + experts (+ optional shared expert);
* per-layer ``(tokens_per_expert, scores)`` pairs are recorded while training
  and turned into the auxiliary loss by :func:`batched_load_balancing_loss`.

Two things differ by design.  The single-device paths never read a count back
to the host (the capacity-0 "dropless by padding" mode of the dropping MoE is
the one exception, as its output *shape* depends on the data).  And the
expert-parallel exchange has two routes: the library all-to-all below, which
mirrors the reference step by step, and the fused peer-memory kernels of
``megablocks_b200.parallel.ep`` that replace the count exchange, both token
all-to-alls and the host round trip when a symmetric workspace is available.
"""

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from megablocks_b200 import ops
from megablocks_b200.layers import common, mlp, mpu, router, sharedexpert_registry
from megablocks_b200.layers.all_to_all import all_to_all
from megablocks_b200.layers.arguments import Arguments
from megablocks_b200.utils.metrics import comm_timer, nvtx_range

_LOAD_BALANCING_LOSS = []


def save_load_balancing_loss(loss) -> None:
    _LOAD_BALANCING_LOSS.append(loss)


def get_load_balancing_loss():
    return _LOAD_BALANCING_LOSS


def clear_load_balancing_loss() -> None:
    _LOAD_BALANCING_LOSS.clear()


def batched_load_balancing_loss(args: Arguments) -> torch.Tensor:
    """``E * w / (L * T * k) * sum_layers <tokens_per_expert, mean_t scores>``."""
    if args.moe_loss_weight == 0:
        return 0.0
    tokens_per_expert, expert_scores = zip(*get_load_balancing_loss())
    layers_here = args.num_layers // args.pipeline_model_parallel_size
    if args.num_layers_per_virtual_pipeline_stage is not None:
        layers_here = args.num_layers_per_virtual_pipeline_stage
    if len(tokens_per_expert) != layers_here:
        raise ValueError(f'Expected {layers_here} token_per_experts but found {len(tokens_per_expert)}.\n'
                         f'num_layers = {args.num_layers}\n'
                         f'pipeline_model_parallel_size = {args.pipeline_model_parallel_size}\n'
                         f'num_layers_per_virtual_pipeline_stage = {args.num_layers_per_virtual_pipeline_stage}')
    if len(expert_scores) != layers_here:
        raise ValueError(f'Expected {layers_here} expert_scores but found {len(expert_scores)}.')
    tokens = expert_scores[0].shape[0]
    for scores, counts in zip(expert_scores, tokens_per_expert):
        assert scores.dim() == 2 and scores.shape == (tokens, args.moe_num_experts)
        assert counts.dim() == 1 and counts.shape[0] == args.moe_num_experts
    scale = (args.moe_num_experts * args.moe_loss_weight) / (args.num_layers * tokens * args.moe_top_k)
    from megablocks_b200.ops import fused
    if tokens != 0 and fused.load_balancing_loss_supported(expert_scores, tokens_per_expert):
        # CUDA: all layers in one reduction kernel (fp32 accumulation whatever `moe_lbl_in_fp32` says),
        # nothing concatenated; the gradient is one broadcast kernel.
        return fused.load_balancing_loss(list(expert_scores), list(tokens_per_expert), scale / tokens)
    # Column means layer by layer, then one concatenation of the [E] vectors: the same numbers as
    # reducing the concatenated [T, L * E] matrix, without materialising it.
    reduced = []
    for layer_scores in expert_scores:
        if args.moe_lbl_in_fp32:
            layer_scores = layer_scores.float()
        reduced.append(layer_scores.mean(dim=0) if tokens != 0 else layer_scores.sum(dim=0))
    scores = torch.cat(reduced)
    counts = torch.cat(tokens_per_expert).to(scores.dtype)
    return scale * torch.dot(counts, scores)


def _as_1d(t: torch.Tensor) -> torch.Tensor:
    return t.view(1) if t.dim() == 0 else t


class ParallelMLP(torch.nn.Module):
    """Experts + permutation (+ expert-parallel exchange) of the token-dropping MoE."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.args = args
        self.num_experts = args.moe_num_experts
        self.top_k = args.moe_top_k
        # Bits of an expert id: the radix sort only looks at these.
        self.sort_end_bit = max((self.num_experts - 1).bit_length(), 1)
        self.mlp = self._build_experts(args)

        if args.bias:
            # The output bias is replicated, not sharded, under expert parallelism.
            self.bias = torch.nn.Parameter(
                torch.zeros(args.hidden_size, device=args.device, dtype=common.dtype(args)))
        else:
            self.register_parameter('bias', None)

        self.forward_fn = self.parallel_forward_once if args.moe_expert_model_parallelism else self.forward_once
        self._ep_workspaces = {}      # activation dtype -> ring of symmetric workspaces of the fused route
        self._ep_calls = 0

    def _build_experts(self, args: Arguments) -> torch.nn.Module:
        return mlp.MLP(args)

    # -- bookkeeping ----------------------------------------------------------
    def expert_capacity(self, tokens: int) -> int:
        world = mpu.get_expert_parallel_world_size(self.args)
        return int(self.args.moe_capacity_factor * (self.top_k * tokens * world / self.num_experts))

    def load_balancing_loss(self, tokens_per_expert: torch.Tensor, expert_scores: torch.Tensor) -> torch.Tensor:
        """Single-layer auxiliary loss (the batched form is used in training)."""
        tokens, num_experts = expert_scores.shape
        assert num_experts == self.num_experts and tokens_per_expert.shape == (num_experts,)
        scale = self.num_experts / (tokens * self.top_k)
        return scale * torch.dot(tokens_per_expert.to(expert_scores.dtype), expert_scores.mean(dim=0))

    def indices_and_bins(self, top_expert: torch.Tensor):
        """``(indices, bin_ids, bins, tokens_per_expert)`` for the flattened expert choice."""
        indices, bin_ids, bins, _, tokens_per_expert = ops.route_plan(top_expert, self.num_experts)
        return indices, bin_ids, bins, tokens_per_expert

    # -- single device --------------------------------------------------------
    def permute_and_compute(self, x, tokens_per_expert, indices, bin_ids, expert_weights, bins, expert_capacity,
                            top_k):
        x = x.reshape(-1, x.shape[-1])
        x = ops.binned_gather(x, indices, bins, expert_capacity, top_k)
        x = self.mlp(x)
        return ops.binned_scatter(x, indices, expert_weights, bins, top_k)

    def forward_once(self, x: torch.Tensor, expert_weights: torch.Tensor, top_experts: torch.Tensor):
        expert_weights = expert_weights.flatten()
        top_experts = top_experts.flatten()
        with torch.no_grad():
            indices, bin_ids, bins, tokens_per_expert = self.indices_and_bins(top_experts)
            tokens = x.numel() // x.shape[-1]
            capacity = self.expert_capacity(tokens)
            if capacity == 0:
                # Dropless by padding: the output shape depends on the data.
                capacity = int(torch.max(tokens_per_expert).item())
        x = self.permute_and_compute(x, tokens_per_expert, indices, bin_ids, expert_weights, bins, capacity,
                                     self.top_k)
        return x, tokens_per_expert

    # -- expert parallel ------------------------------------------------------
    def parallel_forward_once(self, x: torch.Tensor, expert_weights: torch.Tensor, top_experts: torch.Tensor):
        """Expert-parallel forward.

        Library route, step by step: (1) sort copies by expert locally; (2)
        exchange per-expert counts; (3) all-to-all the copies to the ranks that
        own their experts; (4) re-sort the received copies by local expert; (5)
        run the experts; (6) reverse all-to-all; (7) sum hidden-sharding
        replicas; (8) weighted un-permute.  Ranks are laid out expert-major:
        rank ``r`` owns experts ``(r % esd) * epr ..`` and ffn rows
        ``(r // esd) * f/hsd ..``.
        """
        if type(self).permute_and_compute is ParallelMLP.permute_and_compute and self._use_fused_ep(x):
            # Token-dropping experts ([E, h, f] / [E, f, h] weights) over peer memory: the capacity rule
            # of the binned gather is applied by the senders, which know every rank's counts.
            from megablocks_b200.layers.mlp import resolve_dtensor
            copies = top_experts.numel() * mpu.hidden_sharding_degree(self.args)
            return self.fused_parallel_forward_once(x, expert_weights, top_experts, resolve_dtensor(self.mlp.w1),
                                                    resolve_dtensor(self.mlp.w2), None, w1_kn=True,
                                                    expert_capacity=self.expert_capacity(copies))

        args = self.args
        group = args.expert_parallel_group
        world = mpu.get_expert_parallel_world_size(args)
        hsd = mpu.hidden_sharding_degree(args)
        epr = mpu.experts_per_rank(args)

        expert_weights = expert_weights.flatten()
        top_experts = top_experts.flatten()
        with torch.no_grad():
            indices, bin_ids, bins, tokens_per_expert = self.indices_and_bins(top_experts)
            # Every rank that holds a slice of an expert needs that expert's count.
            send_tpe = ops.repeat(tokens_per_expert, (hsd,))
            recv_tpe = torch.empty_like(send_tpe)
            count_handle = dist.all_to_all_single(recv_tpe, send_tpe, group=group, async_op=True)

        x = x.reshape(-1, x.shape[-1])
        x = ops.gather(x, indices, bin_ids, bins, self.top_k)

        with torch.no_grad():
            with comm_timer.region():
                count_handle.wait()
            send_tpe = send_tpe.view(world, epr)
            recv_tpe = recv_tpe.view(world, epr)
            recv_tpe_host = recv_tpe.cpu()
            send_counts = send_tpe.cpu().sum(dim=-1).tolist()
            recv_counts = recv_tpe_host.sum(dim=-1).tolist()
            tokens_received = sum(recv_counts)

        x = ops.repeat(x, (hsd, 1))
        parallel_x, x_handle = all_to_all(x, recv_counts, send_counts, group, async_op=True)

        with torch.no_grad():
            # Received rows are grouped by source rank, then by local expert.
            # Label each with its local expert and sort once more.
            replicate_bins = _as_1d(ops.inclusive_cumsum(recv_tpe.flatten(), 0))
            local_expert = torch.remainder(
                torch.arange(self.num_experts * hsd, dtype=torch.int32, device=indices.device), epr)
            local_expert = ops.replicate(local_expert.unsqueeze(0), replicate_bins, tokens_received).flatten()
            parallel_bin_ids, parallel_indices = ops.sort(local_expert, self.sort_end_bit)
            parallel_tpe = recv_tpe.sum(dim=0, dtype=torch.int)
            parallel_bins = _as_1d(ops.inclusive_cumsum(parallel_tpe, 0))
            capacity = self.expert_capacity(x.shape[0])
            if capacity == 0:
                capacity = int(torch.max(parallel_tpe).item())

        if x_handle is not None:
            with comm_timer.region():
                x_handle.wait()
        parallel_x = self.permute_and_compute(parallel_x, parallel_tpe, parallel_indices, parallel_bin_ids, None,
                                              parallel_bins, capacity, top_k=1)
        x, _ = all_to_all(parallel_x, send_counts, recv_counts, group)
        x = ops.sum(x.view(hsd, -1, args.hidden_size), dim=0)
        x = ops.scatter(x, indices, bin_ids, expert_weights, bins, self.top_k)
        return x, tokens_per_expert.flatten()

    # -- expert parallel over peer memory ----------------------------------------
    def _use_fused_ep(self, x: torch.Tensor) -> bool:
        want = self.args.ep_fused_comm
        if want is False:
            return False
        from megablocks_b200.parallel import ep
        ok = ep.fused_path_available(self.args, x)
        if want is True and not ok:
            raise RuntimeError('ep_fused_comm=True but the peer-memory route cannot serve this layer '
                               '(needs CUDA 16-bit activations, a kernel-known activation, hidden and per-rank ffn '
                               'multiples of 64)')
        return ok

    def fused_parallel_forward_once(self, x, expert_weights, top_experts, w1, w2, v1, w1_kn: bool,
                                    expert_capacity: int):
        """Expert-parallel forward over peer memory (``megablocks_b200.parallel.ep``).

        ``w1`` is ``[E_local, f, h]`` (``w1_kn=False``, dropless layers) or ``[E_local, h, f]``
        (``w1_kn=True``, the token-dropping layer); ``w2`` is ``[E_local, f, h]``.
        ``expert_capacity`` > 0 keeps only the first that many rows every local expert receives,
        counted over the sources in rank order - the rows the reference's binned gather keeps
        (megablocks/layers/moe.py:374-401); the others contribute zeros.

        More ranks than experts: every expert's ffn rows are split over ``hsd`` ranks (hidden
        sharding, megablocks/layers/mpu.py:74-85).  Slice ``h`` of expert ``e`` is treated as the
        virtual expert ``h * E + e``, which rank ``h * esd + e / epr`` owns; every routed copy goes
        to all ``hsd`` slices of its expert, and the weighted combine, which sums all copies of a
        token, adds the slices' partial outputs up.
        """
        from megablocks_b200.ops import gg
        from megablocks_b200.parallel import ep
        args = self.args
        x2d = x.reshape(-1, x.shape[-1])
        expert_weights = expert_weights.flatten()
        hsd = mpu.hidden_sharding_degree(args)
        top_k, num_virtual = self.top_k * hsd, self.num_experts * hsd
        top_experts = top_experts.flatten()
        if hsd > 1:
            shift = torch.arange(hsd, device=top_experts.device, dtype=top_experts.dtype) * self.num_experts
            top_experts = (top_experts.view(-1, 1) + shift).flatten()
            expert_weights = expert_weights.view(-1, 1).expand(-1, hsd).flatten()
        with torch.no_grad():
            indices, bin_ids, bins, _, tokens_per_expert = ops.route_plan(top_experts, num_virtual)
        copies = indices.numel()
        ring = self._ep_workspaces.get(x2d.dtype)
        if ring is None:
            # Created once per activation dtype (a collective: every rank of the group gets here on
            # its first call) and sized for the largest copy count over the group.
            ring = [ep.EpWorkspace(args.expert_parallel_group, num_virtual,
                                   max(copies, int(args.ep_max_copies or 0)), args.hidden_size, x2d.dtype,
                                   x2d.device, capacity_rows=args.ep_capacity_rows)
                    for _ in range(max(1, int(args.ep_inflight_microbatches)))]
            self._ep_workspaces[x2d.dtype] = ring
        workspace = ring[self._ep_calls % len(ring)]
        self._ep_calls += 1
        if copies > workspace.copies:
            raise RuntimeError(
                f'fused expert parallelism: this call routes {copies} copies but the symmetric buffers were sized '
                f'for {workspace.copies}.  Set Arguments.ep_max_copies to the largest tokens x top_k of any rank '
                '(the buffers cannot be regrown inside forward without a collective).')
        out = ep.fused_expert_parallel(x2d, expert_weights.to(x2d.dtype), w1, w2, v1, workspace, indices, bin_ids,
                                       bins, tokens_per_expert, top_k, gg.activation_id(args.activation_fn),
                                       args.memory_optimized_mlp, wgrad_scale=self.mlp.wgrad_scale(), w1_kn=w1_kn,
                                       expert_capacity=int(expert_capacity))
        return out, tokens_per_expert[:self.num_experts]

    def forward(self, x: torch.Tensor, scores: torch.Tensor, expert_weights: torch.Tensor,
                top_experts: torch.Tensor):
        in_shape = x.size()
        x, tokens_per_expert = self.forward_fn(x, expert_weights, top_experts)
        self.last_tokens_per_expert = tokens_per_expert      # device tensor, for load statistics in logs
        if self.training and self.args.moe_loss_weight > 0:
            save_load_balancing_loss((tokens_per_expert, scores))
        x = x.view(in_shape)
        if self.bias is not None:
            if self.args.return_bias:
                return x, self.bias
            return x + self.bias
        return x


class MoE(torch.nn.Module):
    """Router + experts (+ shared expert).  Input ``[..., hidden]``; output has the same shape."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.router = router.LearnedRouter(args)
        self.experts = self._init_experts_mlp(args)
        self.shared_expert = None
        if args.shared_expert:
            self.shared_expert = sharedexpert_registry.get(args)

    def _init_experts_mlp(self, args: Arguments) -> ParallelMLP:
        return ParallelMLP(args)

    def forward(self, x: torch.Tensor):
        # Cast before the permutation: half the bytes to move.
        x = common.cast_if_autocast_enabled(x)
        with nvtx_range('moe.router'):
            scores, expert_weights, top_experts = self.router(x)
        with nvtx_range('moe.experts'):
            out = self.experts(x, scores, expert_weights, top_experts)
        if self.shared_expert is not None:
            out = self.shared_expert.add_experts_sharedexpert(self.shared_expert(x), out)
        return out
