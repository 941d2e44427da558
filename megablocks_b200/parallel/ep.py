"""Expert parallelism over peer memory: fused dispatch / expert GEMMs / combine.

The reference's expert-parallel forward (megablocks/layers/moe.py:237-423) is a
chain of a count all-to-all, a device-to-host copy, two token all-to-alls and a
second sort.  This module replaces all of it for the dropless layers when every
rank of the expert-parallel group sits on one NVLink/NVSwitch domain:

1. every rank maps every peer's workspace (:class:`SymmetricHeap`, CUDA IPC);
2. ``exchange_counts`` gives every rank the full ``[world, experts]`` count matrix
   by remote stores, so senders and receivers derive every offset on the device;
3. ``push`` stores each routed copy straight into its owner's expert-ordered
   buffer and releases one flag per (source, expert);
4. the owner's first expert GEMM starts at once: its TMA-producer warp waits for
   the flags of the expert whose tile it is about to load, so experts are computed
   while later experts are still arriving;
5. ``return_rows`` stores the expert outputs back into the sources' sorted order and
   the source finishes with the weighted top-k reduction.

Backward runs the same exchange with gradients.  No NCCL call, no host
synchronisation and no second sort is involved.  Buffers are sized for the worst
case (every copy of every rank routed to one rank) unless ``capacity_rows`` is
given; exceeding a given capacity is detected on the device and reported through
the status word.

All waits on peers are bounded (two seconds); a wait that expires records a code
that :func:`megablocks_b200.utils.status.check` turns into an exception.
"""

from typing import Any, Dict, Optional, Tuple

import os
import weakref

import torch
import torch.distributed as dist

from megablocks_b200._ext import ext
from megablocks_b200.layers.fused_mlp import mlp_backward, mlp_forward
from megablocks_b200.utils.metrics import comm_timer, nvtx_range

ERR_RETURN_WAIT = 19


def _align(n: int, to: int = 256) -> int:
    return (n + to - 1) // to * to


class SymmetricHeap:
    """A device allocation of equal size on every rank of ``group``, mapped by every peer."""

    def __init__(self, group: dist.ProcessGroup, nbytes: int, device: torch.device):
        self.group, self.nbytes = group, nbytes
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        with torch.cuda.device(device):
            self.local, handle = ext().symm_alloc(nbytes)
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.numpy().tobytes()), group=group)
            self._opened = []
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self.local.data_ptr())
                else:
                    ptr = ext().symm_open(torch.frombuffer(bytearray(h), dtype=torch.uint8))
                    self._opened.append(ptr)
                    ptrs.append(ptr)
            self.peer_base = torch.tensor(ptrs, dtype=torch.int64, device=device)
        dist.barrier(group)

    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def close(self) -> None:
        for ptr in self._opened:
            ext().symm_close(ptr)
        self._opened = []


_LIVE_WORKSPACES = weakref.WeakSet()


def live_workspaces():
    """Every workspace of this process (the trainer's CUDA-graph step advances their device counters)."""
    return list(_LIVE_WORKSPACES)


class EpWorkspace:
    """Per-layer symmetric buffers, flags and sequence numbers of the fused exchange."""

    _shared_backward: Dict[Tuple, SymmetricHeap] = {}

    def __init__(self, group, num_experts: int, copies: int, hidden: int, dtype: torch.dtype, device,
                 capacity_rows: Optional[int] = None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.num_experts, self.epr = num_experts, num_experts // self.world
        # Every rank sizes its buffers for the largest copy count of the group: a rank with a
        # short batch must still be able to receive what the others send.
        agreed = torch.tensor([int(copies)], dtype=torch.int64, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=group)
        copies = int(agreed.item())
        self.copies, self.hidden, self.dtype, self.device = copies, hidden, dtype, device
        self.capacity = int(capacity_rows) if capacity_rows else self.world * copies
        elem = torch.empty((), dtype=dtype).element_size()
        W, E, epr = self.world, num_experts, self.epr
        off = 0

        def take(nbytes):
            nonlocal off
            start = off
            off = _align(off + nbytes)
            return start

        self.off_counts = take(2 * W * E * 4)
        self.off_count_flags = take(W * 4)
        self.off_disp_flags = [take(W * epr * 4), take(W * epr * 4)]
        self.off_ret_flags = [take(W * 4), take(W * 4)]
        self.off_free = take(4)
        self.off_recv_x = take(self.capacity * hidden * elem)
        self.off_ret_y = take(copies * hidden * elem)
        self.heap = SymmetricHeap(group, off, device)
        key = (id(group), self.capacity, copies, hidden, dtype, str(device))
        if key not in EpWorkspace._shared_backward:
            size = _align(self.capacity * hidden * elem) + _align(copies * hidden * elem)
            EpWorkspace._shared_backward[key] = SymmetricHeap(group, size, device)
        self.bwd_heap = EpWorkspace._shared_backward[key]
        self.off_recv_dy = 0
        self.off_ret_dx = _align(self.capacity * hidden * elem)

        self.recv_x = self.heap.view(self.off_recv_x, (self.capacity, hidden), dtype)
        self.ret_y = self.heap.view(self.off_ret_y, (copies, hidden), dtype)
        self.recv_dy = self.bwd_heap.view(self.off_recv_dy, (self.capacity, hidden), dtype)
        self.ret_dx = self.bwd_heap.view(self.off_ret_dx, (copies, hidden), dtype)
        self.seq = 0
        self.released_seq = 0
        # Added by every kernel to the sequence number it is launched with.  Zero as long as the
        # host counts the uses; when the training step is replayed from a CUDA graph (where `seq` is
        # frozen into the recorded launches) the graph adds this workspace's uses per step to it at
        # the end of every replay.
        self.seq_dev = torch.zeros(1, dtype=torch.int32, device=device)
        _LIVE_WORKSPACES.add(self)

    # -- geometry passed to the kernels -------------------------------------------------
    def _layout(self):
        return (self.heap.peer_base, self.world, self.rank, self.num_experts, self.epr, self.capacity,
                self.off_counts, self.off_count_flags)

    def flags(self, offset: int, count: int) -> torch.Tensor:
        return self.heap.view(offset, (count,), torch.int32)

    def next_seq(self) -> int:
        self.seq += 1
        return self.seq

    # -- steps ----------------------------------------------------------------------------
    def exchange_counts(self, tpe: torch.Tensor, seq: int, expert_capacity: int = 0):
        """All-gather of the per-expert copy counts by remote stores.

        Returns ``(counts, recv_bins[experts_per_rank], done)``: ``counts = (kept, routed)``, two
        ``[world * experts]`` matrices - the copies every (rank, expert) pair routed and those that
        survive ``expert_capacity`` rows per expert (0 = no limit: the same numbers) - and ``done``,
        the zeroed completion counters of this call's four push / return kernels.
        """
        E, W = self.num_experts, self.world
        routed = torch.empty(W * E, dtype=torch.int32, device=self.device)
        kept = torch.empty(W * E, dtype=torch.int32, device=self.device)
        recv_bins = torch.empty(self.epr, dtype=torch.int32, device=self.device)
        scratch = torch.empty(2 * E + 2 * W, dtype=torch.int32, device=self.device)
        ext().ep_exchange_counts(tpe, *self._layout(), seq, int(expert_capacity), routed, kept, recv_bins, scratch,
                                 self.seq_dev)
        done = (scratch[:E], scratch[2 * E:2 * E + W], scratch[E:2 * E], scratch[2 * E + W:])
        return (kept, routed), recv_bins, done

    def push(self, x, indices, weights, bins, counts, direction: int, seq: int, top_k: int, done,
             drops: bool = False):
        """Store my routed copies of ``x`` into the owners' receive buffers (0 = forward, 1 = backward).

        With ``drops`` (a capacity limit is on) the return-buffer rows of the copies that are not
        sent are cleared, since no owner will write them.
        """
        kept = counts[0]
        if direction == 0:
            ext().ep_push_rows(x, indices, weights, bins, kept, *self._layout(), self.heap.peer_base,
                               self.off_recv_x, self.off_disp_flags[0], self.off_free, seq, top_k, done,
                               self.ret_y if drops else None, self.seq_dev)
        else:
            ext().ep_push_rows(x, indices, weights, bins, kept, *self._layout(), self.bwd_heap.peer_base,
                               self.off_recv_dy, self.off_disp_flags[1], -1, seq, top_k, done,
                               self.ret_dx if drops else None, self.seq_dev)

    def return_rows(self, y, counts, direction: int, seq: int, done):
        """Store my expert-ordered rows ``y`` back into the sources' sorted order."""
        if direction == 0:
            ext().ep_return_rows(y, counts[0], counts[1], *self._layout(), self.heap.peer_base, self.off_ret_y,
                                 self.off_ret_flags[0], seq, self.copies, done, self.seq_dev)
        else:
            ext().ep_return_rows(y, counts[0], counts[1], *self._layout(), self.bwd_heap.peer_base, self.off_ret_dx,
                                 self.off_ret_flags[1], seq, self.copies, done, self.seq_dev)

    def scatter_args(self, counts, direction: int, seq: int, done):
        """``scatter`` argument of the grouped GEMM: return the output rows to their sources from the epilogue."""
        heap = self.heap if direction == 0 else self.bwd_heap
        off = self.off_ret_y if direction == 0 else self.off_ret_dx
        return ([heap.peer_base, self.heap.peer_base, counts[0], done, counts[1]],
                [off, self.off_ret_flags[direction], self.world, self.rank, self.num_experts, seq, self.copies],
                self.seq_dev)

    def fuse_combine(self) -> bool:
        """Whether the kernel's segment tables can hold this workspace's (expert, rank) pairs."""
        return self.epr * self.world <= 512 and os.environ.get('MB200_EP_FUSED_COMBINE', '1') != '0'

    def wait_return(self, direction: int, seq: int) -> None:
        ext().ep_wait_flags(self.flags(self.off_ret_flags[direction], self.world), self.world, seq, ERR_RETURN_WAIT,
                            self.seq_dev)

    def arrival(self, direction: int, seq: int):
        """``wait`` argument of the grouped GEMM: per-expert arrival flags of the receive buffer."""
        return (self.flags(self.off_disp_flags[direction], self.world * self.epr), self.world, self.epr, seq,
                self.seq_dev)

    def release_receive_buffer(self, seq: int) -> None:
        """Publish that every read of the forward receive buffer of use ``seq`` has been issued."""
        if seq > self.released_seq:
            ext().ep_set_flag(self.flags(self.off_free, 1), seq, self.seq_dev)
            self.released_seq = seq

    def close(self) -> None:
        """Unmap the peers' views of this workspace's own heap (the shared backward heap stays)."""
        self.heap.close()

    def begin_use(self, seq: int) -> None:
        """Called at the start of use ``seq`` of the forward receive buffer.

        Normally the backward pass of use ``seq - 1`` has already released the buffer.  When
        that backward never runs - the forward was the first pass of an activation-checkpointed
        block, whose graph is dropped and recomputed - the release happens here: everything of
        this rank that read the old contents was enqueued on this stream before.  (A backward
        pass of an older use that arrives after a newer forward, as in interleaved pipeline
        schedules, is not supported with one workspace per layer.)
        """
        self.release_receive_buffer(seq - 1)


class _FusedExpertParallel(torch.autograd.Function):
    """dispatch -> expert MLP / GLU -> combine, forward and backward, over peer memory."""

    @staticmethod
    def forward(ctx: Any, x, expert_weights, w1, w2, v1, ws: EpWorkspace, indices, bin_ids, bins, tpe, top_k: int,
                act: int, keep_h: bool, wgrad_scale: float = 1.0, w1_kn: bool = False, expert_capacity: int = 0):
        seq = ws.next_seq()
        ws.begin_use(seq)
        x = x.contiguous()
        tokens = x.shape[0]
        drops = expert_capacity > 0
        with comm_timer.region(), nvtx_range('ep.dispatch'):
            counts, recv_bins, done = ws.exchange_counts(tpe, seq, expert_capacity)
            ws.push(x, indices, None, bins, counts, 0, seq, top_k, done[0], drops)
        fuse = ws.fuse_combine()
        y, saved = mlp_forward(ws.recv_x, w1, w2, v1, recv_bins, act, keep_h, wait=ws.arrival(0, seq),
                               zero_tail=False, rows_hint=ws.copies,
                               scatter=ws.scatter_args(counts, 0, seq, done[1]) if fuse else None, w1_kn=w1_kn)
        with comm_timer.region(), nvtx_range('ep.combine_wait'):
            if not fuse:
                ws.return_rows(y, counts, 0, seq, done[1])
            ws.wait_return(0, seq)
        out = ext().scatter_rows(ws.ret_y, indices, bin_ids, expert_weights, bins, bins, top_k, tokens)
        will_backward = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (x, expert_weights, w1, w2, v1))
        if not will_backward:
            ws.release_receive_buffer(seq)
        z1, z2, h = saved
        tensors = [expert_weights, w1, w2, indices, bin_ids, bins, counts[0], counts[1], recv_bins, z1, done[2],
                   done[3]]
        ctx.glu = v1 is not None
        ctx.keep_h = h is not None
        if ctx.glu:
            tensors += [v1, z2]
        if h is not None:
            tensors.append(h)
        ctx.save_for_backward(*tensors)
        ctx.ws, ctx.seq, ctx.top_k, ctx.act, ctx.tokens = ws, seq, top_k, act, tokens
        ctx.wgrad_scale, ctx.w1_kn, ctx.drops = wgrad_scale, w1_kn, drops
        ctx.mark_non_differentiable()
        return out

    @staticmethod
    def backward(ctx: Any, dout):
        ws, seq, top_k = ctx.ws, ctx.seq, ctx.top_k
        if seq != ws.seq:
            # A newer forward has reused this workspace: its receive buffers and flags no longer
            # belong to this call, and running on would silently produce wrong gradients.
            raise RuntimeError(
                f'fused expert parallelism: backward of use {seq} of a layer workspace after use {ws.seq} '
                'started.  Several forwards of one layer are in flight (pipeline schedule, '
                'forward-forward-backward-backward accumulation, retain_graph): raise '
                'Arguments.ep_inflight_microbatches to their number or set ep_fused_comm=False.')
        saved = list(ctx.saved_tensors)
        expert_weights, w1, w2, indices, bin_ids, bins, kept, routed, recv_bins, z1, done_push, done_ret = saved[:12]
        counts = (kept, routed)
        v1 = z2 = None
        if ctx.glu:
            v1, z2 = saved[12:14]
        h = saved[-1] if ctx.keep_h else None
        dout = dout.contiguous()
        fuse = ws.fuse_combine() and not ctx.w1_kn      # the dx GEMM of the [E, h, f] layout is NT: no fused return
        # d(out)/d(expert rows): each copy's gradient is its token's gradient times its router weight.
        with comm_timer.region(), nvtx_range('ep.dispatch_grad'):
            ws.push(dout, indices, expert_weights, bins, counts, 1, seq, top_k, done_push, ctx.drops)
        dweights = None
        if ctx.needs_input_grad[1]:
            dweights = ext().scatter_wgrad(ws.ret_y, dout, indices, bin_ids, bins, bins, top_k)
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3],
                 ctx.glu and ctx.needs_input_grad[4])
        dxr, dw1, dw2, dv1 = mlp_backward(ws.recv_dy, ws.recv_x, w1, w2, v1, recv_bins, ctx.act, (z1, z2, h),
                                          (True,) + needs[1:], wait=ws.arrival(1, seq), zero_tail=False,
                                          rows_hint=ws.copies,
                                          scatter=ws.scatter_args(counts, 1, seq, done_ret) if fuse else None,
                                          wgrad_scale=ctx.wgrad_scale, w1_kn=ctx.w1_kn)
        # Every read of both receive buffers is enqueued above; only now may peers learn
        # (through the return flags / the free flag) that they can be overwritten.
        with comm_timer.region(), nvtx_range('ep.combine_grad_wait'):
            if not fuse:
                ws.return_rows(dxr, counts, 1, seq, done_ret)
            ws.release_receive_buffer(seq)
            ws.wait_return(1, seq)
        dx = None
        if needs[0]:
            dx = ext().scatter_rows(ws.ret_dx, indices, bin_ids, None, bins, bins, top_k, ctx.tokens)
        return (dx, dweights, dw1, dw2, dv1) + (None,) * 11


def fused_expert_parallel(x, expert_weights, w1, w2, v1, workspace: EpWorkspace, indices, bin_ids, bins, tpe,
                          top_k: int, act: int, memory_optimized: bool, wgrad_scale: float = 1.0,
                          w1_kn: bool = False, expert_capacity: int = 0) -> torch.Tensor:
    """``x[tokens, hidden]`` -> ``out[tokens, hidden]`` through the expert-parallel group of ``workspace``.

    The gradients of ``w1`` / ``w2`` / ``v1`` come out multiplied by ``wgrad_scale``.  ``w1_kn``:
    ``w1`` is ``[E, h, f]`` instead of ``[E, f, h]``.  ``expert_capacity`` > 0 drops every copy past
    that many rows per expert (counted over the sources in rank order); dropped copies contribute
    zeros, forward and backward.
    """
    return _FusedExpertParallel.apply(x, expert_weights, w1, w2, v1, workspace, indices, bin_ids, bins, tpe, top_k,
                                      act, not memory_optimized, wgrad_scale, w1_kn, expert_capacity)


def fused_path_available(args, x: torch.Tensor) -> bool:
    """Whether the peer-memory route can serve this layer call."""
    from megablocks_b200.layers import mpu
    from megablocks_b200.ops import gg
    if not (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)):
        return False
    if gg.activation_id(args.activation_fn) is None:
        return False
    world = mpu.get_expert_parallel_world_size(args)
    experts = args.moe_num_experts
    if world < 2 or (world <= experts and experts % world) or (world > experts and world % experts):
        return False
    if world > experts and args.ffn_hidden_size % (world // experts):
        return False
    if args.hidden_size % 64 or mpu.features_per_rank(args) % 64:
        return False
    return True
