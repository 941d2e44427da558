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
        """``shape`` / ``dtype``: the activations that cross a stage boundary (one micro-batch)."""
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

    def forward_backward(self, run_stage, num_micro_batches: int, loss_fn=None, scale: float = 1.0):
        """GPipe-style schedule: all forwards, then all backwards, activations kept per micro-batch.

        ``run_stage(x, i)`` maps the stage input of micro-batch ``i`` (``None`` on the first stage,
        which fetches its own tokens) to ``(output, auxiliary loss or None)``; the auxiliary loss
        (this stage's load-balancing terms) is back-propagated together with the gradient that
        arrives from the next stage.  The last stage applies ``loss_fn(output, i)``.  Everything
        that is back-propagated is multiplied by ``scale`` (1 / micro-batches, loss scaling).
        Returns the last stage's list of losses (empty elsewhere).
        """
        inputs, outputs, auxes, losses = [], [], [], []
        for i in range(num_micro_batches):
            x = None
            if not self.is_first:
                x, _ = self.exchange(recv_prev=True)
                x.requires_grad_(True)
            y, aux = run_stage(x, i)
            if self.is_last:
                losses.append(loss_fn(y, i))
            else:
                self.exchange(send_next=y.detach())
            inputs.append(x)
            outputs.append(y)
            auxes.append(aux)
        for i in reversed(range(num_micro_batches)):
            roots, grads = [], []
            if self.is_last:
                roots.append(losses[i] * scale)
                grads.append(None)
            else:
                _, grad = self.exchange(recv_next=True)
                roots.append(outputs[i])
                grads.append(grad)
            if auxes[i] is not None and torch.is_tensor(auxes[i]) and auxes[i].requires_grad:
                roots.append(auxes[i] * scale)
                grads.append(None)
            torch.autograd.backward(roots, grads)
            if not self.is_first:
                self.exchange(send_prev=inputs[i].grad)
            outputs[i] = auxes[i] = None      # free the micro-batch's graph
        return losses
