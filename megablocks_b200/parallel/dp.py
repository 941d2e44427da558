"""Data-parallel gradient reduction overlapped with backward, and ZeRO-1 sharding.

The reference leaves data parallelism to its outer trainer (Megatron-LM
``--DDP-impl local``, exp/dmoe/dmoe_125m_8gpu.sh:145) and only tags expert
weights with ``expert_model_parallel`` so that trainer can skip them
(megablocks/layers/mpu.py:31-52).  This module is the native counterpart:

* :class:`FlatBuffer` re-homes the replicated ("dense") parameters and their
  gradients in two contiguous buffers, laid out in reverse registration order
  so the gradients that backward produces first sit at the front;
* :class:`GradReducer` cuts the buffer into buckets and, from autograd's
  post-accumulate hooks, launches each bucket's collective on a side stream the
  moment its last gradient lands - all-reduce (plain DP) or reduce-scatter
  (ZeRO-1: every rank then owns one slice of every bucket);
* with ZeRO-1 the optimizer updates only the owned slices and the updated
  parameters are all-gathered bucket by bucket.

Buckets are sized for launch latency and overlap (NVSwitch gives every pair of
GPUs full bandwidth, so there is no per-link reason to make them large).

Two backends move the bytes.  ``'peer'`` (the default on CUDA when every rank of the
group can map its peers' memory): the gradient buffer lives in a symmetric heap and one
kernel of this library per bucket (``csrc/dp_comm.cu``) reduces it with peer loads and
stores over NVLink - ready flags, a reduce of the rank's own slice, stores into every
rank's slice, done flags - without any NCCL call.  ``'nccl'``: ``all_reduce`` /
``reduce_scatter_tensor``, kept as the baseline and for CPU (gloo) ranks.
"""

from typing import List, Optional, Sequence

import os

import torch
import torch.distributed as dist


def _align(n: int, to: int) -> int:
    return (n + to - 1) // to * to


class PeerScalarSum:
    """Sum of one fp32 value over the group by the peer-memory reducer kernel (no NCCL call).

    Used for the squared gradient norm: rank 0 of the group adds the ranks' values in rank order and
    stores the sum into every rank's buffer, so all ranks clip with bitwise the same coefficient.
    The kernel's closing handshake guarantees that no peer still reads this rank's buffer when the
    call returns on the stream, so the next call may overwrite it.
    """

    def __init__(self, group: dist.ProcessGroup, device):
        from megablocks_b200.parallel.ep import SymmetricHeap
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        flag_bytes = _align(self.world * 4, 256)
        self._off_ready, self._off_done = 256, 256 + flag_bytes
        self._heap = SymmetricHeap(group, 256 + 2 * flag_bytes, device)
        self._heap.local.zero_()
        self.buf = self._heap.view(0, (4,), torch.float32)
        self._ticket = torch.zeros(1, dtype=torch.int32, device=device)
        self.seq = 0
        self.seq_dev = torch.zeros(1, dtype=torch.int32, device=device)   # see GradReducer.seq_dev
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def __call__(self, value: torch.Tensor) -> None:
        """``value`` (one fp32 element on this device) becomes the sum over the group, in place."""
        from megablocks_b200._ext import ext
        self.buf[:1].copy_(value.reshape(1))
        self.seq += 1
        ext().dp_allreduce(self.buf, self._heap.peer_base, self.world, self.rank, 0, self._off_ready, self._off_done,
                           0, 4, 0, self.seq, 1.0, False, self._ticket, 1, self.seq_dev)
        value.reshape(1).copy_(self.buf[:1])


class FlatBuffer:
    """Contiguous parameter and gradient storage for a list of same-dtype parameters."""

    def __init__(self, params: Sequence[torch.nn.Parameter], granule: int = 8):
        self.params = list(reversed(list(params)))   # backward order
        assert self.params, 'FlatBuffer needs at least one parameter'
        dtype, device = self.params[0].dtype, self.params[0].device
        self.offsets, total = [], 0
        for p in self.params:
            assert p.dtype == dtype and p.device == device
            self.offsets.append(total)
            total += _align(p.numel(), 8)
        self.numel = _align(total, granule)
        self.param = torch.zeros(self.numel, dtype=dtype, device=device)
        self.grad = torch.zeros(self.numel, dtype=dtype, device=device)
        for p, off in zip(self.params, self.offsets):
            view = self.param[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grad[off:off + p.numel()].view_as(p)

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p, off in zip(self.params, self.offsets):   # re-attach in case something dropped the view
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + off * self.grad.element_size():
                p.grad = self.grad[off:off + p.numel()].view_as(p)


class GradReducer:
    """Bucketed gradient collective launched from backward hooks on a side stream."""

    def __init__(self, flat: FlatBuffer, group: Optional[dist.ProcessGroup], bucket_bytes: int = 32 << 20,
                 shard: bool = False, backend: str = 'auto', ctas: int = 16):
        self.flat, self.group, self.shard = flat, group, shard
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        elem = flat.grad.element_size()
        granule = self.world * 8
        target = max(granule, _align(bucket_bytes // elem, granule))
        # Bucket boundaries fall on parameter boundaries (a hook fires per parameter).
        self.buckets: List[List[int]] = []   # [start, end, first param idx, last param idx + 1]
        start, first = 0, 0
        for i, (p, off) in enumerate(zip(flat.params, flat.offsets)):
            end = off + _align(p.numel(), 8)
            last = i == len(flat.params) - 1
            if end - start >= target or last:
                end = flat.numel if last else end
                self.buckets.append([start, end, first, i + 1])
                start, first = end, i + 1
        if shard:
            for b in self.buckets:
                assert (b[1] - b[0]) % granule == 0 or b is self.buckets[-1]
            assert flat.numel % granule == 0
        self._bucket_of = {}
        for bi, (_, _, lo, hi) in enumerate(self.buckets):
            for i in range(lo, hi):
                self._bucket_of[i] = bi
        self._pending = [hi - lo for (_, _, lo, hi) in self.buckets]
        self._remaining = list(self._pending)
        self._launched = [False] * len(self.buckets)
        self._stream = torch.cuda.Stream() if flat.grad.is_cuda else None
        self._works = []
        # With gradient accumulation only the last micro-batch's backward may start the collectives:
        # the trainer clears `active` for the earlier ones.
        self.active = True
        self.backend = self._pick_backend(backend)
        self.ctas = int(ctas)
        self.seq = 0
        if self.backend == 'peer':
            self._init_peer()
        for i, p in enumerate(flat.params):
            p.register_post_accumulate_grad_hook(self._make_hook(i))

    # -- peer-memory backend -------------------------------------------------------
    def _pick_backend(self, backend: str) -> str:
        if backend not in ('auto', 'peer', 'nccl'):
            raise ValueError(f"backend must be 'auto', 'peer' or 'nccl', got {backend!r}")
        backend = os.environ.get('MB200_DP_BACKEND', backend)
        usable = self.flat.grad.is_cuda and self.flat.grad.dtype in (torch.bfloat16, torch.float16, torch.float32)
        if backend == 'peer' and not usable:
            raise RuntimeError("the 'peer' gradient reducer needs CUDA gradients")
        if backend == 'auto':
            backend = 'peer' if usable else 'nccl'
        return backend

    def _init_peer(self) -> None:
        """Re-home the gradient buffer in a symmetric heap that every rank of the group maps."""
        from megablocks_b200.parallel.ep import SymmetricHeap
        flat = self.flat
        grad_bytes = _align(flat.numel * flat.grad.element_size(), 256)
        flag_bytes = _align(len(self.buckets) * self.world * 4, 256)
        self._off_grad, self._off_ready, self._off_done = 0, grad_bytes, grad_bytes + flag_bytes
        self._heap = SymmetricHeap(self.group, grad_bytes + 2 * flag_bytes, flat.grad.device)
        self._heap.local.zero_()
        new_grad = self._heap.view(0, (flat.numel,), flat.grad.dtype)
        new_grad.copy_(flat.grad)
        flat.grad = new_grad
        flat.zero_grad()                       # re-attaches every p.grad view to the new storage
        self._tickets = torch.zeros(len(self.buckets), dtype=torch.int32, device=flat.grad.device)
        # Added by the kernel to the step number it is launched with; the trainer's CUDA-graph step
        # (whose recorded launches carry a frozen `seq`) adds one to it at the end of every replay.
        self.seq_dev = torch.zeros(1, dtype=torch.int32, device=flat.grad.device)
        torch.cuda.synchronize(flat.grad.device)
        dist.barrier(self.group)               # nobody launches before every heap is zeroed

    def _launch_peer(self, bi: int) -> None:
        from megablocks_b200._ext import ext
        s, e = self.buckets[bi][:2]
        ext().dp_allreduce(self.flat.grad, self._heap.peer_base, self.world, self.rank, self._off_grad,
                           self._off_ready, self._off_done, s, e - s, bi, self.seq, 1.0 / self.world, self.shard,
                           self._tickets[bi:bi + 1], self.ctas, self.seq_dev)

    # -- shard geometry (ZeRO-1) --------------------------------------------------
    def shard_range(self, bucket: int):
        s, e = self.buckets[bucket][:2]
        n = (e - s) // self.world
        return s + self.rank * n, s + (self.rank + 1) * n

    def _make_hook(self, index: int):
        def hook(_param):
            if not self.active:
                return
            bi = self._bucket_of[index]
            self._remaining[bi] -= 1
            if self._remaining[bi] == 0:
                self._launch(bi)
        return hook

    def _launch(self, bi: int) -> None:
        if self._launched[bi]:
            return
        if self.backend == 'peer' and not any(self._launched):
            self.seq += 1        # first bucket of this step
        self._launched[bi] = True
        s, e = self.buckets[bi][:2]
        grad = self.flat.grad[s:e]
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(self._stream)
        else:
            ctx = _NullContext()
        with ctx:
            if self.backend == 'peer':
                self._launch_peer(bi)
            elif self.shard and grad.is_cuda:
                lo, hi = self.shard_range(bi)
                out = self.flat.grad[lo:hi]
                work = dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.AVG, group=self.group, async_op=True)
                self._works.append((work, grad))
            elif grad.is_cuda:
                work = dist.all_reduce(grad, op=dist.ReduceOp.AVG, group=self.group, async_op=True)
                self._works.append((work, grad))
            else:
                # CPU ranks (gloo): no AVG and no reduce-scatter; sum everything, then divide.
                dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group)
                grad.div_(self.world)

    def reset(self) -> None:
        """Forget a step that was abandoned half way (no bucket counts as launched, none as pending)."""
        self._works.clear()
        self._remaining = list(self._pending)
        self._launched = [False] * len(self.buckets)
        self.active = True

    def finish(self) -> None:
        """Launch whatever backward did not trigger, then make the current stream wait for all buckets."""
        for bi in range(len(self.buckets)):
            self._launch(bi)
        for work, _ in self._works:
            work.wait()
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)
        self._works.clear()
        self._remaining = list(self._pending)
        self._launched = [False] * len(self.buckets)

    def gather_params(self) -> None:
        """ZeRO-1: all-gather the updated parameter slices of every bucket."""
        assert self.shard
        for bi, (s, e, _, _) in enumerate(self.buckets):
            lo, hi = self.shard_range(bi)
            mine = self.flat.param[lo:hi].clone()
            if mine.is_cuda:
                dist.all_gather_into_tensor(self.flat.param[s:e], mine, group=self.group)
            else:
                pieces = list(self.flat.param[s:e].chunk(self.world))
                dist.all_gather(pieces, mine, group=self.group)


class _NullContext:

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
