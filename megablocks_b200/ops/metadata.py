"""Integer metadata ops: sort, histogram, prefix sums, topology, replicate.

Each op has two implementations behind one entry point: a few lines of plain
PyTorch for CPU tensors (also the oracle in the tests) and a hand-written
sm_100a kernel in ``csrc/metadata.cu`` for CUDA tensors.  Semantics follow the
reference ops (megablocks/ops/sort.py:26-38, histogram.py:20-27,
cumsum.py:20-51, round_up.py:7-14, topology.py:20-45, replicate.py:19-36,
repeat.py:7-10, sum.py:6-9), including their quirks:

* ``sort`` returns the permutation in the *key* dtype and orders by the low
  ``end_bit`` bits only;
* a 1-D ``cumsum`` of a single element returns a 0-dim tensor;
* ``topology`` returns int16 block-column ids.
"""

from typing import Any, Optional, Tuple

import torch

from megablocks_b200._ext import ext

_INT_BITS = {torch.int16: 16, torch.int32: 32, torch.int64: 64}


# ----------------------------------------------------------------------------
# sort
# ----------------------------------------------------------------------------
def sort(x: torch.Tensor, end_bit: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable key/index sort of a 1-D integer tensor on bits ``[0, end_bit)``.

    Returns ``(sorted_keys, permutation)``; ``permutation[i]`` is the position
    in ``x`` of the element now at ``i`` and has the dtype of ``x``.
    """
    if x.dtype not in _INT_BITS:
        raise ValueError(f'sort expects int16/int32/int64, got {x.dtype}')
    if x.dim() != 1:
        raise ValueError('sort expects a 1-D tensor')
    width = _INT_BITS[x.dtype]
    if end_bit is None:
        end_bit = width
    end_bit = int(min(max(end_bit, 1), width))
    if x.is_cuda:
        keys, perm = ext().sort_pairs(x.contiguous(), end_bit)
        return keys, perm
    if end_bit >= width:
        radix_key = x
    else:
        radix_key = x.to(torch.int64) & ((1 << end_bit) - 1)
    order = torch.argsort(radix_key, stable=True)
    return x[order], order.to(x.dtype)


# ----------------------------------------------------------------------------
# histogram
# ----------------------------------------------------------------------------
def histogram(x: torch.Tensor, num_bins: int) -> torch.Tensor:
    """Counts of the values ``0 .. num_bins-1`` per row; int32 output."""
    if x.dtype not in _INT_BITS:
        raise ValueError(f'histogram expects int16/int32/int64, got {x.dtype}')
    if x.dim() not in (1, 2):
        raise ValueError('histogram expects a 1-D or 2-D tensor')
    flat = x.dim() == 1
    rows = x.view(1, -1) if flat else x
    if x.is_cuda:
        out = ext().histogram(rows.contiguous(), int(num_bins))
    else:
        out = torch.zeros(rows.shape[0], num_bins, dtype=torch.int32)
        for r in range(rows.shape[0]):
            vals = rows[r].to(torch.int64)
            vals = vals[(vals >= 0) & (vals < num_bins)]
            out[r] = torch.bincount(vals, minlength=num_bins).to(torch.int32)
    return out.view(-1) if flat else out


# ----------------------------------------------------------------------------
# prefix sums
# ----------------------------------------------------------------------------
def _cumsum(x: torch.Tensor, dim: int, exclusive: bool) -> torch.Tensor:
    if x.dim() == 1:
        if dim != 0:
            raise ValueError('a 1-D cumsum runs along dim 0')
        return _cumsum(x.view(1, -1), 1, exclusive).squeeze()
    if x.dim() != 2 or dim != 1:
        raise ValueError('cumsum expects a 2-D tensor scanned along dim 1')
    if x.is_cuda and x.dtype in _INT_BITS:
        return ext().cumsum(x.contiguous(), bool(exclusive))
    inclusive = torch.cumsum(x, dim=1).to(x.dtype)
    return inclusive - x if exclusive else inclusive


def exclusive_cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    return _cumsum(x, dim, True)


def inclusive_cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    return _cumsum(x, dim, False)


def round_up(x: torch.Tensor, value: int) -> torch.Tensor:
    """Round every element of an int32 tensor up to a multiple of ``value``."""
    if not isinstance(value, int):
        raise ValueError('round_up takes an integer multiple')
    if x.dtype != torch.int32:
        raise ValueError('round_up expects an int32 tensor')
    return torch.div(x + (value - 1), value, rounding_mode='trunc') * value


# ----------------------------------------------------------------------------
# topology
# ----------------------------------------------------------------------------
def topology(padded_bins: torch.Tensor, block_size: int, output_block_rows: int,
             output_block_columns: int) -> torch.Tensor:
    """Block-column ids of the block-diagonal expert matrix.

    Row-blocks ``[padded_bins[e-1]/B, padded_bins[e]/B)`` belong to expert
    ``e`` and hold column-blocks ``e*C .. e*C+C-1`` (``C`` = blocks per expert).
    Row-blocks past ``padded_bins[-1]`` are left zero.  Returns int16 of length
    ``rows * C``.
    """
    if padded_bins.dim() != 1 or padded_bins.dtype != torch.int32:
        raise ValueError('padded_bins must be a 1-D int32 tensor')
    rows, cols = int(output_block_rows), int(output_block_columns)
    if padded_bins.is_cuda:
        return ext().topology(padded_bins.contiguous(), int(block_size), rows, cols)
    out = torch.zeros(rows, cols, dtype=torch.int16)
    ends = torch.div(padded_bins, block_size, rounding_mode='trunc').to(torch.int64)
    starts = torch.cat([ends.new_zeros(1), ends[:-1]])
    row_ids = torch.arange(rows)
    col_ids = torch.arange(cols)
    for e in range(padded_bins.numel()):
        mask = (row_ids >= starts[e]) & (row_ids < ends[e])
        out[mask] = (e * cols + col_ids).to(torch.int16)
    return out.view(-1)


# ----------------------------------------------------------------------------
# replicate
# ----------------------------------------------------------------------------
def _replicate_forward(x: torch.Tensor, bins: torch.Tensor, num_outputs: int) -> torch.Tensor:
    if x.is_cuda:
        return ext().replicate_forward(x.contiguous(), bins.contiguous(), int(num_outputs))
    ends = bins.to(torch.int64)
    counts = ends - torch.cat([ends.new_zeros(1), ends[:-1]])
    out = torch.repeat_interleave(x, counts, dim=1)
    if out.shape[1] < num_outputs:
        pad = x.new_zeros(x.shape[0], num_outputs - out.shape[1])
        out = torch.cat([out, pad], dim=1)
    return out[:, :num_outputs].contiguous()


def _replicate_backward(grad: torch.Tensor, bins: torch.Tensor) -> torch.Tensor:
    if grad.is_cuda:
        return ext().replicate_backward(grad.contiguous(), bins.contiguous())
    ends = bins.to(torch.int64)
    starts = torch.cat([ends.new_zeros(1), ends[:-1]])
    acc = torch.cat([grad.new_zeros(grad.shape[0], 1, dtype=torch.float32),
                     torch.cumsum(grad.float(), dim=1)], dim=1)
    return (acc[:, ends] - acc[:, starts]).to(grad.dtype)


class _Replicate(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, bins: torch.Tensor, num_outputs: int):
        ctx.save_for_backward(bins)
        return _replicate_forward(x, bins, num_outputs)

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor):
        bins, = ctx.saved_tensors
        return _replicate_backward(grad.contiguous(), bins), None, None


def replicate(x: torch.Tensor, bins: torch.Tensor, num_outputs: int) -> torch.Tensor:
    """Run-length expansion: ``out[b, bins[i-1]:bins[i]] = x[b, i]``.

    The backward pass is the matching segmented sum.
    """
    if x.dim() != 2 or bins.dim() != 1 or x.shape[1] != bins.shape[0]:
        raise ValueError('replicate expects x[batch, num_bins] and bins[num_bins]')
    return _Replicate.apply(x, bins, num_outputs)


def repeat(x: torch.Tensor, tiling) -> torch.Tensor:
    """``x.repeat(tiling)`` that returns ``x`` itself when every factor is 1."""
    if all(int(t) == 1 for t in tiling):
        return x
    return x.repeat(*tiling)


def sum(x: torch.Tensor, dim: int = 0) -> torch.Tensor:  # noqa: A001 - public name of the op
    """Sum over ``dim``; a size-1 ``dim`` is squeezed without arithmetic."""
    if x.shape[dim] == 1:
        return x.squeeze(dim=dim)
    return x.sum(dim=dim)
