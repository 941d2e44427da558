"""Learned top-k router and the router z-loss.

Behaviour matches the reference router (megablocks/layers/router.py:10-114):
optional multiplicative input jitter while training, a bias-free linear map to
expert logits, softmax over experts, top-k selection (ties resolve to the
lowest expert id), optional p-norm normalisation of the k weights and an
optional forced round-robin assignment for benchmarking.  Logits are recorded
in a module-level list when the z-loss is enabled; the trainer reads them with
:func:`batched_router_zloss` and must call :func:`clear_router_zloss` each step.

On CUDA the softmax / top-k / normalisation chain and its backward run as one
kernel each (``csrc/router.cu``); the logits GEMM is a plain library GEMM.
"""

import warnings
from typing import Any

import torch

from megablocks_b200.layers import common
from megablocks_b200.layers.arguments import Arguments

_ROUTER_LOGITS = []


def _save_router_logits(logits: torch.Tensor, args: Arguments) -> None:
    if args.moe_zloss_weight == 0:
        return
    _ROUTER_LOGITS.append(logits)


def clear_router_zloss() -> None:
    _ROUTER_LOGITS.clear()


def batched_router_zloss(args: Arguments):
    """One z-loss value per recorded layer: ``w * mean_t(logsumexp_e(logits)^2)``."""
    if args.moe_zloss_weight == 0:
        warnings.warn('Call to batched_router_zloss, but moe_zloss_weight=0')
        return 0
    per_layer = []
    for logits in _ROUTER_LOGITS:
        if args.moe_zloss_in_fp32:
            logits = logits.float()
        per_layer.append(torch.logsumexp(logits, dim=1).square().mean())
    return args.moe_zloss_weight * torch.stack(per_layer)


class _UniformExpertAssignment(torch.autograd.Function):
    """Replace the chosen experts by 0,1,..,E-1,0,1,.. (perfectly balanced load)."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, num_experts: int):
        ids = torch.arange(x.numel(), dtype=x.dtype, device=x.device)
        return torch.remainder(ids, num_experts).view(x.shape)

    @staticmethod
    def backward(ctx: Any, grad):  # pragma: no cover - integer output
        return None, None


_uniform_expert_assignment = _UniformExpertAssignment.apply


class _FusedTopK(torch.autograd.Function):
    """softmax -> top-k -> optional p-norm normalisation, one CUDA kernel each way."""

    @staticmethod
    def forward(ctx: Any, logits: torch.Tensor, top_k: int, norm_p: float):
        from megablocks_b200._ext import ext
        scores, weights, experts = ext().router_topk_forward(logits.contiguous(), top_k, float(norm_p))
        ctx.save_for_backward(scores, weights, experts)
        ctx.norm_p = float(norm_p)
        ctx.mark_non_differentiable(experts)
        return scores, weights, experts

    @staticmethod
    def backward(ctx: Any, dscores, dweights, _dexperts):
        from megablocks_b200._ext import ext
        scores, weights, experts = ctx.saved_tensors
        if dscores is None:
            dscores = torch.zeros_like(scores)
        if dweights is None:
            dweights = torch.zeros_like(weights)
        dlogits = ext().router_topk_backward(scores, weights, experts, dscores.contiguous(),
                                             dweights.contiguous(), ctx.norm_p)
        return dlogits, None, None


class LearnedRouter(torch.nn.Module):
    """``Linear(hidden -> experts)`` + softmax + top-k.  Returns ``(scores, weights, experts)``."""

    def __init__(self, args: Arguments):
        super().__init__()
        self.args = args
        # The router weight is replicated on every expert-parallel rank: each
        # rank routes its own tokens and needs all expert logits.
        self.layer = torch.nn.Linear(
            args.hidden_size,
            args.moe_num_experts,
            bias=False,
            dtype=common.dtype(args),
            device=args.device,
        )
        args.init_method(self.layer.weight)

    def jitter(self, x: torch.Tensor) -> torch.Tensor:
        eps = self.args.moe_jitter_eps
        noise = torch.rand(x.size(), dtype=x.dtype, device=x.device)
        return (1.0 - eps) + noise * (2.0 * eps)

    def _top_k(self, scores: torch.Tensor):
        if self.args.moe_top_k == 1:
            return scores.max(dim=-1, keepdim=True)
        return torch.topk(scores, self.args.moe_top_k, dim=-1)

    def _select(self, logits: torch.Tensor):
        args = self.args
        norm_p = args.moe_normalize_expert_weights
        fused_ok = (logits.is_cuda and logits.dtype in (torch.float16, torch.bfloat16, torch.float32)
                    and args.moe_num_experts <= 1024 and args.moe_top_k <= 8
                    and (not norm_p or float(norm_p) in (1.0, 2.0)))
        if fused_ok:
            return _FusedTopK.apply(logits, args.moe_top_k, float(norm_p) if norm_p else 0.0)
        scores = logits.softmax(dim=-1)
        weights, experts = self._top_k(scores)
        if norm_p:
            weights = weights / torch.norm(weights, p=norm_p, dim=-1, keepdim=True)
        return scores, weights, experts

    def forward(self, x: torch.Tensor):
        if self.training and self.args.moe_jitter_eps is not None:
            x = x * self.jitter(x)
        logits = self.layer(x.reshape(-1, x.shape[-1]))
        _save_router_logits(logits, self.args)
        scores, weights, experts = self._select(logits)
        if self.args.uniform_expert_assignment:
            experts = _uniform_expert_assignment(experts, self.args.moe_num_experts)
        return scores, weights, experts
