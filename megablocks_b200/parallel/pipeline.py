"""Pipeline-parallel stage plumbing on overlapped NCCL point-to-point.

The reference has no pipeline code: it only validates how many per-layer
load-balancing terms a pipeline stage should have collected
(megablocks/layers/moe.py:39-60) and leaves send / recv to Megatron-LM.  This
module provides that missing piece for stand-alone use: a stage owns a slice of
the transformer blocks, receives activations from the previous stage, sends its
output to the next one (and gradients the other way), with the transfers issued
as batched ``isend`` / ``irecv`` so they overlap with compute of the neighbouring
micro-batch.  MoE layers inside a stage keep their own expert-parallel group.
"""

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def stage_layers(num_layers: int, num_stages: int, stage: int) -> range:
    """Contiguous block of layer indices owned by ``stage`` (earlier stages take the remainder)."""
    base, extra = divmod(num_layers, num_stages)
    start = stage * base + min(stage, extra)
    return range(start, start + base + (1 if stage < extra else 0))


class PipelineStage:

    def __init__(self, group: Optional[dist.ProcessGroup], shape: Sequence[int], dtype: torch.dtype, device):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.shape, self.dtype, self.device = tuple(shape), dtype, device
        self.is_first = self.rank == 0
        self.is_last = self.rank == self.world - 1

    def _peer(self, offset: int) -> int:
        return dist.get_global_rank(self.group, self.rank + offset) if self.group is not None else self.rank + offset

    def _buffer(self) -> torch.Tensor:
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    def exchange(self, send_next: Optional[torch.Tensor] = None, send_prev: Optional[torch.Tensor] = None,
                 recv_prev: bool = False, recv_next: bool = False) -> Tuple[Optional[torch.Tensor], ...]:
        """One batched round of sends and receives; returns ``(from_prev, from_next)``."""
        ops: List[dist.P2POp] = []
        from_prev = from_next = None
        if recv_prev and not self.is_first:
            from_prev = self._buffer()
            ops.append(dist.P2POp(dist.irecv, from_prev, self._peer(-1), self.group))
        if send_next is not None and not self.is_last:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self._peer(+1), self.group))
        if recv_next and not self.is_last:
            from_next = self._buffer()
            ops.append(dist.P2POp(dist.irecv, from_next, self._peer(+1), self.group))
        if send_prev is not None and not self.is_first:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self._peer(-1), self.group))
        if ops:
            for work in dist.batch_isend_irecv(ops):
                work.wait()
        return from_prev, from_next

    def forward_backward(self, blocks: torch.nn.Module, micro_batches: Sequence[torch.Tensor], loss_fn=None):
        """GPipe-style schedule: all forwards, then all backwards, activations kept per micro-batch.

        ``blocks(x)`` maps the stage input to its output; the first stage receives the
        elements of ``micro_batches`` itself, the last stage applies ``loss_fn(output)``
        and returns the list of losses.
        """
        inputs, outputs, losses = [], [], []
        for mb in micro_batches:
            if self.is_first:
                x = mb
            else:
                x, _ = self.exchange(recv_prev=True)
                x.requires_grad_(True)
            y = blocks(x)
            if self.is_last:
                losses.append(loss_fn(y))
            else:
                self.exchange(send_next=y.detach())
            inputs.append(x)
            outputs.append(y)
        for i in reversed(range(len(micro_batches))):
            if self.is_last:
                losses[i].backward()
            else:
                _, grad = self.exchange(recv_next=True)
                outputs[i].backward(grad)
            if not self.is_first:
                self.exchange(send_prev=inputs[i].grad)
        return losses
