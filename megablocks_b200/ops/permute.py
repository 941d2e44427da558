"""Token permutation ops: gather / scatter and their padded and binned forms.

Notation: ``T`` tokens, ``k`` experts per token, ``n = T*k`` routed copies.
Copy ``c`` belongs to token ``c // k``.  ``indices[i]`` is the copy placed at
sorted position ``i`` and ``bin_ids[i]`` its expert; ``bins`` is the inclusive
prefix sum of copies per expert and ``padded_bins`` the same after rounding
every expert up to a multiple of the block size.

* ``gather``-type ops copy token rows into expert order,
  ``out[row(i)] = x[indices[i] // k] (* weights[indices[i]])``;
* ``scatter``-type ops are the inverse and reduce the ``k`` copies of a token,
  ``out[t] = sum_s weights[t*k+s] * x[row(pos(t*k+s))]``.

The reduction over ``k`` is done in token order inside one kernel, so results
are bitwise reproducible (no floating-point atomics).  Products are formed in
fp32 and rounded once.  Reference semantics: megablocks/ops/gather.py:12-38,
scatter.py:13-72, padded_gather.py:12-55, padded_scatter.py:12-98,
binned_gather.py:12-37, binned_scatter.py:12-59 and the row-copy kernels in
megablocks/backend/kernels.py:34-518.

CPU tensors run the PyTorch statements below; CUDA tensors run the vectorised
kernels of ``csrc/permute.cu``.
"""

from typing import Any, Optional

import torch

from megablocks_b200._ext import ext
from megablocks_b200.utils import debug


# ----------------------------------------------------------------------------
# Shared index arithmetic (CPU path / oracle).
# ----------------------------------------------------------------------------
def _starts(ends: torch.Tensor) -> torch.Tensor:
    ends = ends.to(torch.int64)
    return torch.cat([ends.new_zeros(1), ends[:-1]])


def _dest_rows(bin_ids: torch.Tensor, bins: torch.Tensor, padded_bins: torch.Tensor) -> torch.Tensor:
    """Row of every sorted position in the (padded) expert-ordered buffer."""
    e = bin_ids.to(torch.int64)
    pos = torch.arange(e.numel(), device=e.device)
    return _starts(padded_bins)[e] + (pos - _starts(bins)[e])


def _scaled(rows: torch.Tensor, weights: Optional[torch.Tensor], copy_ids: torch.Tensor, dtype) -> torch.Tensor:
    if weights is None:
        return rows.to(dtype)
    return (rows.float() * weights.float()[copy_ids].unsqueeze(1)).to(dtype)


def _sum_top_k(tmp: torch.Tensor, tokens: int, top_k: int) -> torch.Tensor:
    if top_k == 1:
        return tmp
    return tmp.view(tokens, top_k, -1).float().sum(dim=1).to(tmp.dtype)


# ----------------------------------------------------------------------------
# Kernels behind the padded / unpadded ops.
# ----------------------------------------------------------------------------
def _gather_rows(x, indices, bin_ids, weights, bins, padded_bins, top_k, out_rows):
    debug.check_routing(indices, bin_ids, bins, padded_bins, top_k, x.shape[0], out_rows)
    if x.is_cuda:
        return ext().gather_rows(x, indices, bin_ids, weights, bins, padded_bins, top_k, out_rows)
    copy_ids = indices.to(torch.int64)
    out = x.new_zeros(out_rows, x.shape[1])
    rows = _dest_rows(bin_ids, bins, padded_bins)
    out[rows] = _scaled(x[copy_ids // top_k], weights, copy_ids, x.dtype)
    return out


def _scatter_rows(x, indices, bin_ids, weights, bins, padded_bins, top_k):
    tokens = indices.numel() // top_k
    debug.check_routing(indices, bin_ids, bins, padded_bins, top_k, tokens, x.shape[0])
    if x.is_cuda:
        return ext().scatter_rows(x, indices, bin_ids, weights, bins, padded_bins, top_k, tokens)
    copy_ids = indices.to(torch.int64)
    rows = _dest_rows(bin_ids, bins, padded_bins)
    tmp = x.new_zeros(tokens * top_k, x.shape[1])
    tmp[copy_ids] = _scaled(x[rows], weights, copy_ids, x.dtype)
    return _sum_top_k(tmp, tokens, top_k)


def _scatter_wgrad(x, grad, indices, bin_ids, bins, padded_bins, top_k):
    """d(loss)/d(weights): one dot product of an expert row with its token's grad."""
    debug.check_routing(indices, bin_ids, bins, padded_bins, top_k, grad.shape[0], x.shape[0])
    if x.is_cuda:
        return ext().scatter_wgrad(x, grad, indices, bin_ids, bins, padded_bins, top_k)
    copy_ids = indices.to(torch.int64)
    rows = _dest_rows(bin_ids, bins, padded_bins)
    out = torch.zeros(indices.numel(), dtype=x.dtype)
    out[copy_ids] = (x[rows].float() * grad[copy_ids // top_k].float()).sum(dim=1).to(x.dtype)
    return out


def _check_routing(indices, bin_ids, bins, padded_bins=None):
    for name, t in (('indices', indices), ('bin_ids', bin_ids), ('bins', bins), ('padded_bins', padded_bins)):
        if t is None:
            continue
        if t.dim() != 1 or t.dtype != torch.int32:
            raise ValueError(f'{name} must be a 1-D int32 tensor')
    if indices.numel() != bin_ids.numel():
        raise ValueError('indices and bin_ids must have the same length')


def _autocast(x):
    if x is not None and x.is_cuda and torch.is_autocast_enabled('cuda') and x.is_floating_point():
        return x.to(torch.get_autocast_dtype('cuda'))
    return x


class _Gather(torch.autograd.Function):
    """Token order -> expert order; backward is the unweighted scatter."""

    @staticmethod
    def forward(ctx: Any, x, indices, bin_ids, bins, padded_bins, top_k, out_rows):
        x = _autocast(x)
        ctx.save_for_backward(indices, bin_ids, bins, padded_bins)
        ctx.top_k = top_k
        return _gather_rows(x.contiguous(), indices, bin_ids, None, bins, padded_bins, top_k, out_rows)

    @staticmethod
    def backward(ctx: Any, grad):
        indices, bin_ids, bins, padded_bins = ctx.saved_tensors
        dx = _scatter_rows(grad.contiguous(), indices, bin_ids, None, bins, padded_bins, ctx.top_k)
        return dx, None, None, None, None, None, None


class _Scatter(torch.autograd.Function):
    """Expert order -> token order with router weights and the top-k sum."""

    @staticmethod
    def forward(ctx: Any, x, indices, bin_ids, weights, bins, padded_bins, top_k):
        x = _autocast(x)
        weights = _autocast(weights)
        need_wgrad = weights is not None and weights.requires_grad
        saved = [indices, bin_ids, bins, padded_bins]
        if weights is not None:
            saved.append(weights)
        if need_wgrad:
            saved.append(x)
        ctx.save_for_backward(*saved)
        ctx.has_weights = weights is not None
        ctx.need_wgrad = need_wgrad
        ctx.top_k = top_k
        ctx.x_rows = x.shape[0]
        return _scatter_rows(x.contiguous(), indices, bin_ids, weights, bins, padded_bins, top_k)

    @staticmethod
    def backward(ctx: Any, grad):
        grad = grad.contiguous()
        saved = ctx.saved_tensors
        indices, bin_ids, bins, padded_bins = saved[:4]
        weights = saved[4] if ctx.has_weights else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _gather_rows(grad, indices, bin_ids, weights, bins, padded_bins, ctx.top_k, ctx.x_rows)
        dw = None
        if ctx.need_wgrad:
            x = saved[-1]
            dw = _scatter_wgrad(x, grad, indices, bin_ids, bins, padded_bins, ctx.top_k)
        return dx, None, None, dw, None, None, None


def gather(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, bins: torch.Tensor,
           top_k: int) -> torch.Tensor:
    """``out[i] = x[indices[i] // top_k]`` for every sorted position ``i``."""
    _check_routing(indices, bin_ids, bins)
    return _Gather.apply(x, indices, bin_ids, bins, bins, top_k, indices.numel())


def scatter(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, weights: Optional[torch.Tensor],
            bins: torch.Tensor, top_k: int) -> torch.Tensor:
    """Inverse of :func:`gather` with optional per-copy weights; sums the ``top_k`` copies."""
    _check_routing(indices, bin_ids, bins)
    return _Scatter.apply(x, indices, bin_ids, weights, bins, bins, top_k)


def padded_gather(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor, bins: torch.Tensor,
                  padded_bins: torch.Tensor, top_k: int, num_rows: Optional[int] = None) -> torch.Tensor:
    """Gather into the block-padded layout; pad rows are zero.

    ``num_rows`` is the height of the output.  When it is omitted the exact
    height ``padded_bins[-1]`` is read back from the device (one host sync, as
    in the reference); the layers pass a static upper bound instead so that the
    forward pass never waits for the GPU.
    """
    _check_routing(indices, bin_ids, bins, padded_bins)
    if num_rows is None:
        num_rows = int(padded_bins[-1].item())
    return _Gather.apply(x, indices, bin_ids, bins, padded_bins, top_k, int(num_rows))


def padded_scatter(x: torch.Tensor, indices: torch.Tensor, bin_ids: torch.Tensor,
                   weights: Optional[torch.Tensor], bins: torch.Tensor, padded_bins: torch.Tensor,
                   top_k: int) -> torch.Tensor:
    """Inverse of :func:`padded_gather` with optional weights and the top-k sum."""
    _check_routing(indices, bin_ids, bins, padded_bins)
    return _Scatter.apply(x, indices, bin_ids, weights, bins, padded_bins, top_k)


# ----------------------------------------------------------------------------
# Binned (capacity-limited) ops for the token-dropping MoE.
# ----------------------------------------------------------------------------
def _binned_slots(indices, bins, capacity):
    """(expert, slot, keep-mask) of every sorted position."""
    ends = bins.to(torch.int64)
    starts = _starts(bins)
    pos = torch.arange(indices.numel(), device=indices.device)
    expert = torch.searchsorted(ends, pos, right=True)
    expert = expert.clamp_(max=ends.numel() - 1)
    slot = pos - starts[expert]
    keep = (slot < capacity) & (pos < ends[-1])
    return expert, slot, keep


def _binned_gather_rows(x, indices, weights, bins, capacity, top_k):
    if x.is_cuda:
        return ext().binned_gather_rows(x, indices, weights, bins, capacity, top_k)
    num_experts = bins.numel()
    out = x.new_zeros(num_experts, capacity, x.shape[1])
    expert, slot, keep = _binned_slots(indices, bins, capacity)
    copy_ids = indices.to(torch.int64)[keep]
    out[expert[keep], slot[keep]] = _scaled(x[copy_ids // top_k], weights, copy_ids, x.dtype)
    return out


def _binned_scatter_rows(x, indices, weights, bins, top_k):
    tokens = indices.numel() // top_k
    if x.is_cuda:
        return ext().binned_scatter_rows(x, indices, weights, bins, top_k, tokens)
    capacity = x.shape[1]
    expert, slot, keep = _binned_slots(indices, bins, capacity)
    copy_ids = indices.to(torch.int64)[keep]
    tmp = x.new_zeros(tokens * top_k, x.shape[2])
    tmp[copy_ids] = _scaled(x[expert[keep], slot[keep]], weights, copy_ids, x.dtype)
    return _sum_top_k(tmp, tokens, top_k)


def _binned_scatter_wgrad(x, grad, indices, bins, top_k):
    if x.is_cuda:
        return ext().binned_scatter_wgrad(x, grad, indices, bins, top_k)
    capacity = x.shape[1]
    expert, slot, keep = _binned_slots(indices, bins, capacity)
    copy_ids = indices.to(torch.int64)[keep]
    out = torch.zeros(indices.numel(), dtype=x.dtype)
    out[copy_ids] = (x[expert[keep], slot[keep]].float() * grad[copy_ids // top_k].float()).sum(dim=1).to(x.dtype)
    return out


class _BinnedGather(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x, indices, bins, bin_size, top_k):
        x = _autocast(x)
        ctx.save_for_backward(indices, bins)
        ctx.top_k = top_k
        return _binned_gather_rows(x.contiguous(), indices, None, bins, bin_size, top_k)

    @staticmethod
    def backward(ctx: Any, grad):
        indices, bins = ctx.saved_tensors
        dx = _binned_scatter_rows(grad.contiguous(), indices, None, bins, ctx.top_k)
        return dx, None, None, None, None


class _BinnedScatter(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x, indices, weights, bins, top_k):
        x = _autocast(x)
        weights = _autocast(weights)
        need_wgrad = weights is not None and weights.requires_grad
        saved = [indices, bins]
        if weights is not None:
            saved.append(weights)
        if need_wgrad:
            saved.append(x)
        ctx.save_for_backward(*saved)
        ctx.has_weights = weights is not None
        ctx.need_wgrad = need_wgrad
        ctx.top_k = top_k
        ctx.bin_size = x.shape[1]
        return _binned_scatter_rows(x.contiguous(), indices, weights, bins, top_k)

    @staticmethod
    def backward(ctx: Any, grad):
        grad = grad.contiguous()
        saved = ctx.saved_tensors
        indices, bins = saved[:2]
        weights = saved[2] if ctx.has_weights else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _binned_gather_rows(grad, indices, weights, bins, ctx.bin_size, ctx.top_k)
        dw = None
        if ctx.need_wgrad:
            dw = _binned_scatter_wgrad(saved[-1], grad, indices, bins, ctx.top_k)
        return dx, None, dw, None, None


def binned_gather(x: torch.Tensor, indices: torch.Tensor, bins: torch.Tensor, bin_size: int,
                  top_k: int) -> torch.Tensor:
    """``out[e, j] = x[indices[bins[e-1] + j] // top_k]`` for ``j < min(bin_size, count_e)``; rest zero."""
    _check_routing(indices, indices, bins)
    if x.dim() != 2:
        raise ValueError('binned_gather expects x[tokens, hidden]')
    return _BinnedGather.apply(x, indices, bins, int(bin_size), top_k)


def binned_scatter(x: torch.Tensor, indices: torch.Tensor, weights: Optional[torch.Tensor], bins: torch.Tensor,
                   top_k: int) -> torch.Tensor:
    """Inverse of :func:`binned_gather`; copies that were dropped contribute zero."""
    _check_routing(indices, indices, bins)
    if x.dim() != 3 or x.shape[0] != bins.numel():
        raise ValueError('binned_scatter expects x[num_experts, bin_size, hidden]')
    return _BinnedScatter.apply(x, indices, weights, bins, top_k)
