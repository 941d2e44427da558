"""Differentiable variable-split all-to-all on a process group.

Reference: megablocks/layers/all_to_all.py:8-54.  ``all_to_all(x, recv, send,
group, async_op)`` returns ``(out, handle)``; its backward runs the exchange in
the opposite direction with the split lists swapped.  This is the library
(NCCL / gloo) route; the fused peer-memory route lives in
``megablocks_b200.parallel``.
"""

from typing import Any, List, Optional

import torch
import torch.distributed as dist

from megablocks_b200.utils.metrics import comm_timer


def _exchange(x, out_splits, in_splits, group, async_op):
    out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    x = x.contiguous()
    if async_op:    # the caller's wait() is the exposed part and is timed there
        handle = dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits,
                                        group=group, async_op=True)
        return out, handle
    with comm_timer.region():
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out, None


class AllToAllOp(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x, output_split_sizes: List[int], input_split_sizes: List[int], group, async_op: bool):
        ctx.input_shape = x.shape
        ctx.output_split_sizes = output_split_sizes
        ctx.input_split_sizes = input_split_sizes
        ctx.group = group
        return _exchange(x, output_split_sizes, input_split_sizes, group, async_op)

    @staticmethod
    def backward(ctx: Any, grad, _handle):
        if not ctx.needs_input_grad[0]:
            return None, None, None, None, None
        out, _ = _exchange(grad, ctx.input_split_sizes, ctx.output_split_sizes, ctx.group, False)
        return out, None, None, None, None


def all_to_all(x: torch.Tensor, output_split_sizes: List[int], input_split_sizes: List[int],
               group: Optional[dist.ProcessGroup], async_op: bool = False):
    return AllToAllOp.apply(x, output_split_sizes, input_split_sizes, group, async_op)
