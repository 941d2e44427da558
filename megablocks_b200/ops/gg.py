"""Grouped GEMM: one matrix product per expert over a ragged batch of rows.

This takes the place of the external ``grouped_gemm`` package the reference
calls (call sites: megablocks/layers/mlp.py:414-523, glu.py:84-205).  Groups
are described by ``bins``: an int32 device tensor holding the inclusive prefix
sum of rows per expert, so no row count ever has to be copied to the host.

Layouts (``n`` rows in total, ``E`` groups):

=========  ======================  =========================  ============
trans_a    a                       b                          result
=========  ======================  =========================  ============
False      ``[n, K]``              ``[E, K, N]`` (NN) or      ``[n, N]``
                                   ``[E, N, K]`` (trans_b)
True       ``[n, M]``              ``[n, N]``                 ``[E, M, N]``
=========  ======================  =========================  ============

With ``trans_a`` the contraction runs over each group's rows (ragged K); a
group without rows yields a zero matrix.  On CUDA all of these run the
tcgen05/TMEM kernel of ``csrc/grouped_gemm.cu``, optionally with a fused
epilogue (activation, activation backward, GLU product, GLU backward).  On
CPU they run per-group ``torch.matmul`` in fp32, which is also the oracle.
"""

import os
from functools import partial
from typing import Any, Callable, Optional

import torch
import torch.nn.functional as F

from megablocks_b200._ext import ext
from megablocks_b200.utils import debug

# Epilogue kinds understood by the kernel.
EPI_NONE = 0      # c = acc
EPI_ACT = 1       # c = acc, out2 = act(acc)
EPI_DACT = 2      # c = acc * act'(aux1), out2 = act(aux1)
EPI_GLU = 3       # c = acc, out2 = act(aux1) * acc
EPI_DGLU = 4      # c = acc * aux2 * act'(aux1), out2 = acc * act(aux1), out3 = act(aux1) * aux2
EPI_ADD = 5       # c = acc + aux1
EPI_GLU_DUAL = 6  # two weight operands: c = a b2^T, out2 = act(a b^T) * c, out3 = a b^T

ACT_IDENTITY = 0
ACT_GELU_TANH = 1
ACT_SILU = 2
ACT_RELU = 3
ACT_GELU_ERF = 4

_ACT_NAMES = {
    'identity': ACT_IDENTITY,
    'gelu_tanh': ACT_GELU_TANH,
    'silu': ACT_SILU,
    'relu': ACT_RELU,
    'gelu': ACT_GELU_ERF,
}


# CTA-pair (cta_group::2) kernel selection: 1 = whenever supported, anything else = never (the
# default: measured against the single-CTA kernel it does not win on any shape tried).  Overridable
# for experiments with MB200_GEMM_PAIR or per call (`pair=`).
_PAIR_MODE = int(os.environ.get('MB200_GEMM_PAIR', '0'))


def activation_id(fn: Optional[Callable]) -> Optional[int]:
    """Kernel id of a known activation callable; ``None`` for anything else."""
    if fn is None:
        return ACT_IDENTITY
    if isinstance(fn, str):
        return _ACT_NAMES.get(fn)
    if isinstance(fn, partial):
        if fn.func is F.gelu and not fn.args:
            approx = fn.keywords.get('approximate', 'none')
            if set(fn.keywords) <= {'approximate'}:
                return ACT_GELU_TANH if approx == 'tanh' else ACT_GELU_ERF
        return None
    if fn is F.gelu:
        return ACT_GELU_ERF
    if fn is F.silu:
        return ACT_SILU
    if fn is F.relu or fn is torch.relu:
        return ACT_RELU
    if isinstance(fn, torch.nn.GELU):
        return ACT_GELU_TANH if fn.approximate == 'tanh' else ACT_GELU_ERF
    if isinstance(fn, torch.nn.SiLU):
        return ACT_SILU
    if isinstance(fn, torch.nn.ReLU):
        return ACT_RELU
    return None


def act_forward(z: torch.Tensor, act: int) -> torch.Tensor:
    if act == ACT_IDENTITY:
        return z
    if act == ACT_GELU_TANH:
        return F.gelu(z, approximate='tanh')
    if act == ACT_SILU:
        return F.silu(z)
    if act == ACT_RELU:
        return F.relu(z)
    if act == ACT_GELU_ERF:
        return F.gelu(z)
    raise ValueError(f'unknown activation id {act}')


def act_derivative(z: torch.Tensor, act: int) -> torch.Tensor:
    """d act(z) / dz evaluated in the dtype of ``z`` (callers pass fp32)."""
    if act == ACT_IDENTITY:
        return torch.ones_like(z)
    if act == ACT_GELU_TANH:
        c = 0.7978845608028654
        inner = c * (z + 0.044715 * z * z * z)
        t = torch.tanh(inner)
        return 0.5 * (1 + t) + 0.5 * z * (1 - t * t) * c * (1 + 3 * 0.044715 * z * z)
    if act == ACT_SILU:
        s = torch.sigmoid(z)
        return s * (1 + z * (1 - s))
    if act == ACT_RELU:
        return (z > 0).to(z.dtype)
    if act == ACT_GELU_ERF:
        cdf = 0.5 * (1 + torch.erf(z * 0.7071067811865476))
        pdf = torch.exp(-0.5 * z * z) * 0.3989422804014327
        return cdf + z * pdf
    raise ValueError(f'unknown activation id {act}')


def bins_from_batch_sizes(batch_sizes: torch.Tensor, device) -> torch.Tensor:
    """Inclusive prefix sum (int32, on ``device``) of a per-group row count tensor."""
    return torch.cumsum(batch_sizes.to(torch.int64), dim=0).to(dtype=torch.int32).to(device, non_blocking=True)


# ----------------------------------------------------------------------------
# CPU implementation (oracle).
# ----------------------------------------------------------------------------
def _bounds(bins: torch.Tensor):
    ends = [int(v) for v in bins.tolist()]
    starts = [0] + ends[:-1]
    return list(zip(starts, ends))


def _cpu_grouped_gemm(a, b, bins, trans_a, trans_b, num_groups):
    if trans_a:
        out = torch.zeros(num_groups, a.shape[1], b.shape[1], dtype=torch.float32, device=a.device)
        for e, (s, t) in enumerate(_bounds(bins)):
            if t > s:
                out[e] = a[s:t].float().t() @ b[s:t].float()
        return out
    n_out = b.shape[1] if trans_b else b.shape[2]
    out = torch.zeros(a.shape[0], n_out, dtype=torch.float32, device=a.device)
    for e, (s, t) in enumerate(_bounds(bins)):
        if t > s:
            w = b[e].float()
            out[s:t] = a[s:t].float() @ (w.t() if trans_b else w)
    return out


def _cpu_epilogue(acc, epilogue, act, aux1, aux2, dtype):
    if epilogue == EPI_NONE:
        return acc.to(dtype), None, None
    if epilogue == EPI_ACT:
        c = acc.to(dtype)
        return c, act_forward(c.float(), act).to(dtype), None
    if epilogue == EPI_DACT:
        z = aux1.float()
        return (acc * act_derivative(z, act)).to(dtype), act_forward(z, act).to(dtype), None
    if epilogue == EPI_GLU:
        c = acc.to(dtype)
        return c, (act_forward(aux1.float(), act) * c.float()).to(dtype), None
    if epilogue == EPI_DGLU:
        z1, z2 = aux1.float(), aux2.float()
        a1 = act_forward(z1, act)
        return ((acc * z2 * act_derivative(z1, act)).to(dtype), (acc * a1).to(dtype), (a1 * z2).to(dtype))
    if epilogue == EPI_ADD:
        return (acc + aux1.float()).to(dtype), None, None
    raise ValueError(f'unknown epilogue {epilogue}')


# ----------------------------------------------------------------------------
# Raw (non-autograd) entry point.
# ----------------------------------------------------------------------------
class GradNormSink:
    """Squared norms of weight gradients, taken by the GEMMs that produce them.

    While a sink is installed (:func:`set_grad_norm_sink`), every weight-gradient launch that asks
    for it (``grouped_gemm(..., trans_a=True, grad_norm=True)``) adds the sum of squares of its
    output to a float32 slot of its own and the sink remembers ``output address -> slot``.  The
    trainer later looks its gradient tensors up by address: a tensor it finds needs no second pass
    over its elements for the clipping norm; one it does not find (autograd copied or accumulated
    it) is summed the ordinary way, so nothing is ever counted twice.
    """

    def __init__(self, device, slots: int = 1024):
        self.slots = torch.zeros(slots, dtype=torch.float32, device=device)
        self._by_address = {}

    def begin(self) -> None:
        self.slots.zero_()
        self._by_address.clear()

    def _next(self):
        i = len(self._by_address)
        return (i, self.slots[i:i + 1]) if i < self.slots.numel() else (None, None)

    def _record(self, out: torch.Tensor, slot: int) -> None:
        self._by_address[out.data_ptr()] = (slot, out.numel())

    def lookup(self, grad: torch.Tensor):
        """Slot index of the launch that wrote exactly this tensor, or ``None``."""
        hit = self._by_address.get(grad.data_ptr())
        return hit[0] if hit is not None and hit[1] == grad.numel() else None


_GRAD_NORM_SINK: Optional[GradNormSink] = None


def set_grad_norm_sink(sink: Optional[GradNormSink]) -> None:
    global _GRAD_NORM_SINK
    _GRAD_NORM_SINK = sink


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, bins: torch.Tensor, *, trans_a: bool = False,
                 trans_b: bool = False, epilogue: int = EPI_NONE, act: int = ACT_IDENTITY,
                 aux1: Optional[torch.Tensor] = None, aux2: Optional[torch.Tensor] = None,
                 want_out2: bool = True, want_out3: bool = True, num_groups: Optional[int] = None,
                 c: Optional[torch.Tensor] = None, zero_tail: bool = True, wait=None,
                 rows_hint: int = 0, scatter=None, alpha: float = 1.0, pair: Optional[int] = None,
                 a2: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None, grad_norm: bool = False):
    """Run one grouped GEMM; returns ``(c, out2, out3)`` (unused outputs are ``None``).

    ``bins`` may describe fewer rows than ``a`` has (the block-padded layout
    allocates an upper bound); rows past ``bins[-1]`` are written as zero.
    ``c`` optionally supplies the output buffer of the main result.  ``zero_tail=False``
    leaves those trailing rows untouched (used with worst-case sized buffers).
    ``wait = (flags, count, stride, seq)`` makes the kernel's load warp wait, per
    group ``g``, until ``flags[s * stride + g] >= seq`` for every ``s < count``: the
    rows of ``a`` are then being delivered by peer GPUs (expert-parallel dispatch).
    ``rows_hint`` is the expected number of occupied rows when ``a`` is a worst-case sized
    buffer (kept for kernel-selection heuristics; currently unused).
    ``scatter = ([data_bases, flag_bases, counts, done], [data_off, flag_off, world, rank, experts,
    seq, return_rows])`` (NN layout) stores every output row into the return buffer of the rank it came from
    instead of ``c`` and releases that rank's flag after its last row: the expert-parallel combine
    fused into the GEMM epilogue.  The returned ``c`` is then empty.
    ``alpha`` multiplies every accumulator before the epilogue (e.g. the 1 / expert-parallel-world
    factor of expert weight gradients, applied for free instead of by a separate pass).
    ``b2`` with ``epilogue=EPI_GLU_DUAL`` (``trans_b`` layout): the GLU forward in one launch - every
    tile multiplies its rows of ``a`` with the matching rows of ``b`` and of ``b2``; returns
    ``(a b2^T, act(a b^T) * (a b2^T), a b^T)``.  ``a2`` and ``b2`` without ``trans_b``: the contraction
    runs over ``a x b`` and then ``a2 x b2`` into one accumulator, ``c = a b + a2 b2`` (the GLU input
    gradient in one launch).
    ``pair`` overrides the kernel choice for this call: 1 = CTA pairs (``cta_group::2``, 256-row
    tiles) whenever the problem allows, 0 = single-CTA kernel, ``None`` = the module default.
    ``grad_norm`` (with ``trans_a``): the output is a weight gradient; if a :class:`GradNormSink` is
    installed the epilogue also adds the output's sum of squares to a slot of the sink.
    """
    if num_groups is None:
        num_groups = bins.numel()
    debug.check_groups(bins, a.shape[0])
    if a.is_cuda and ext().grouped_gemm_supported(a, b, bool(trans_a), bool(trans_b), int(num_groups)):
        flags, count, stride, seq = wait[:4] if wait is not None else (None, 0, 0, 0)
        # Optional device counter that the kernel adds to the sequence numbers of `wait` / `scatter`.
        seq_base = wait[4] if wait is not None and len(wait) > 4 else (
            scatter[2] if scatter is not None and len(scatter) > 2 else None)
        pair_mode = _PAIR_MODE if pair is None else int(pair)
        sink, slot, slot_view = _GRAD_NORM_SINK, None, None
        if grad_norm and sink is not None and trans_a and pair_mode != 1:
            slot, slot_view = sink._next()
        outs = ext().grouped_gemm(a, b, bins, bool(trans_a), bool(trans_b), int(epilogue), int(act), aux1, aux2,
                                  bool(want_out2), bool(want_out3), int(num_groups), c, bool(zero_tail), flags,
                                  int(count), int(stride), int(seq), int(rows_hint), pair_mode,
                                  scatter[0] if scatter is not None else None,
                                  scatter[1] if scatter is not None else [], float(alpha), a2, b2, slot_view,
                                  seq_base)
        if slot is not None:
            sink._record(outs[0], slot)
        return outs
    if scatter is not None:
        raise RuntimeError('grouped_gemm: the fused combine needs the CUDA kernel (unsupported shape or dtype)')
    if wait is not None:
        raise RuntimeError('grouped_gemm: peer-arrival waits need the CUDA kernel (unsupported shape or dtype)')
    # Shapes or dtypes the tensor-core kernel does not take (fp32 inputs, rows that
    # are not a multiple of 8 elements, more than 1024 groups) and every CPU tensor:
    # per-group matmuls in fp32.  On CUDA this reads the group sizes back to the host.
    acc = _cpu_grouped_gemm(a, b, bins, trans_a, trans_b, num_groups)
    if a2 is not None:
        acc = acc + _cpu_grouped_gemm(a2, b2, bins, trans_a, trans_b, num_groups)
    if alpha != 1.0:
        acc = acc * alpha
    if epilogue == EPI_GLU_DUAL:
        z1 = acc.to(a.dtype)
        z2 = (_cpu_grouped_gemm(a, b2, bins, trans_a, trans_b, num_groups) * alpha).to(a.dtype)
        out = (z2, (act_forward(z1.float(), act) * z2.float()).to(a.dtype), z1)
        last = int(bins[-1])
        for t in out:
            if last < t.shape[0]:
                t[last:] = 0
        return out
    out, out2, out3 = _cpu_epilogue(acc, epilogue, act, aux1, aux2, a.dtype)
    if not trans_a:
        # Rows past the last bin belong to no group: defined as zero.
        last = int(bins[-1])
        for t in (out, out2, out3):
            if t is not None and last < t.shape[0]:
                t[last:] = 0
    if c is not None:
        c.copy_(out)
        out = c
    return out, (out2 if want_out2 else None), (out3 if want_out3 else None)


# ----------------------------------------------------------------------------
# Autograd-aware gmm with the call signature of the grouped_gemm package.
# ----------------------------------------------------------------------------
class _GroupedGemm(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, a, b, bins, trans_b):
        ctx.save_for_backward(a, b, bins)
        ctx.trans_b = trans_b
        out, _, _ = grouped_gemm(a.contiguous(), b.contiguous(), bins, trans_b=trans_b)
        return out

    @staticmethod
    def backward(ctx: Any, grad):
        a, b, bins = ctx.saved_tensors
        grad = grad.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da, _, _ = grouped_gemm(grad, b, bins, trans_b=not ctx.trans_b)
        if ctx.needs_input_grad[1]:
            if ctx.trans_b:   # b is [E, N, K]: db_e = grad_e^T @ a_e
                db, _, _ = grouped_gemm(grad, a, bins, trans_a=True, num_groups=b.shape[0])
            else:             # b is [E, K, N]: db_e = a_e^T @ grad_e
                db, _, _ = grouped_gemm(a, grad, bins, trans_a=True, num_groups=b.shape[0])
            db = db.to(b.dtype)
        return da, db, None, None


def gmm(a: torch.Tensor, b: torch.Tensor, batch_sizes: torch.Tensor, trans_b: bool = False) -> torch.Tensor:
    """``grouped_gemm.ops.gmm`` replacement.

    ``batch_sizes`` holds rows per group (any integer dtype, host or device);
    pass a device tensor to stay free of host synchronisation.
    """
    bins = bins_from_batch_sizes(batch_sizes, a.device)
    return _GroupedGemm.apply(a, b, bins, trans_b)


def gmm_bins(a: torch.Tensor, b: torch.Tensor, bins: torch.Tensor, trans_b: bool = False) -> torch.Tensor:
    """Like :func:`gmm` but takes the inclusive prefix sum directly."""
    return _GroupedGemm.apply(a, b, bins, trans_b)


class _Backend:
    """Mirror of ``grouped_gemm.backend``: raw, non-differentiable ``gmm``."""

    @staticmethod
    def gmm(a, b, batch_sizes, trans_a=False, trans_b=False, c=None):
        bins = bins_from_batch_sizes(batch_sizes, a.device)
        out, _, _ = grouped_gemm(a, b, bins, trans_a=trans_a, trans_b=trans_b, c=c,
                                 num_groups=batch_sizes.numel())
        return out


backend = _Backend()
