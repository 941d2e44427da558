"""Fused Adam(W) with fp32 master weights for 16-bit parameters.

The model computes with bf16/fp16 parameters; the optimizer keeps an fp32 copy
and the two Adam moments in flat buffers and updates everything - moments,
master weights and the 16-bit shadow - in ONE kernel launch per parameter
group (``csrc/optim.cu``), reading the gradient-clipping coefficient from
device memory so a step never synchronises with the host.  On CPU tensors the
same arithmetic runs in PyTorch (used by the CPU tests and as the oracle).

This is the optimizer the reference delegates to Megatron-LM (bf16 parameters,
fp32 main copies, Adam, ``--clip-grad 1.0``: exp/dmoe/dmoe_125m_8gpu.sh:65-72,144).
"""

import math
from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch

from megablocks_b200._ext import ext

_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_RECORD = np.dtype([('param', '<u8'), ('grad', '<u8'), ('master', '<u8'), ('exp_avg', '<u8'), ('exp_avg_sq', '<u8'),
                    ('numel', '<i8'), ('norm_weight', '<f4'), ('pad', '<i4')])
_CHUNK = 65536


def _align(n: int, to: int = 8) -> int:
    return (n + to - 1) // to * to


class FusedAdam:
    """Adam / AdamW over a list of tensors with flat fp32 state.

    ``params`` are the tensors the model uses (any float dtype); ``grads_of``
    returns the matching gradient tensors at step time (default: ``p.grad``).
    ``norm_weights`` weights each tensor's contribution to the global gradient
    norm (e.g. ``1/replicas`` for tensors replicated over a group whose squared
    norms are summed).
    """

    def __init__(self, params: Iterable[torch.Tensor], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, norm_weights: Optional[Sequence[float]] = None):
        self.params: List[torch.Tensor] = [p for p in params]
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        # Optional CUDA float32 tensor {lr, bias1, bias2}: when set, the kernel reads the three values
        # from it instead of taking them as launch arguments (used by the trainer's CUDA-graph step,
        # whose recorded launches must follow the schedule).
        self.hyper: Optional[torch.Tensor] = None
        self.norm_weights = list(norm_weights) if norm_weights is not None else [1.0] * len(self.params)
        if not self.params:
            self.device = torch.device('cpu')
            self.offsets = []
            self.master = self.exp_avg = self.exp_avg_sq = torch.zeros(0)
            return
        self.device = self.params[0].device
        self.dtype = self.params[0].dtype
        assert all(p.device == self.device and p.dtype == self.dtype for p in self.params)
        offsets, total = [], 0
        for p in self.params:
            offsets.append(total)
            total += _align(p.numel())
        self.offsets = offsets
        self.master = torch.zeros(total, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        for p, off in zip(self.params, offsets):
            self.master[off:off + p.numel()].copy_(p.detach().reshape(-1))
        if self.device.type == 'cuda':
            self._init_tables()

    # -- tables (CUDA) ----------------------------------------------------------
    def _init_tables(self):
        assert ext().adam_record_size() == _RECORD.itemsize
        rec = np.zeros(len(self.params), dtype=_RECORD)
        blocks = []
        self._block_start = []          # first job of every tensor (plus the total at the end)
        for i, (p, off) in enumerate(zip(self.params, self.offsets)):
            self._block_start.append(len(blocks))
            rec[i]['param'] = p.data_ptr()
            rec[i]['master'] = self.master.data_ptr() + 4 * off
            rec[i]['exp_avg'] = self.exp_avg.data_ptr() + 4 * off
            rec[i]['exp_avg_sq'] = self.exp_avg_sq.data_ptr() + 4 * off
            rec[i]['numel'] = p.numel()
            rec[i]['norm_weight'] = self.norm_weights[i]
            for c in range((p.numel() + _CHUNK - 1) // _CHUNK):
                blocks.append((i, c))
        self._block_start.append(len(blocks))
        self._records = rec
        self._blocks = torch.tensor(blocks, dtype=torch.int32).reshape(-1, 2).to(self.device)
        self._host_ring = [torch.empty(rec.nbytes, dtype=torch.uint8).pin_memory() for _ in range(4)]
        self._table = torch.empty(rec.nbytes, dtype=torch.uint8, device=self.device)
        self._ring_pos = 0

    def _upload_table(self, grads: Sequence[torch.Tensor]):
        rec = self._records
        for i, (p, g) in enumerate(zip(self.params, grads)):
            assert g.is_contiguous() and g.numel() == p.numel()
            rec[i]['grad'] = g.data_ptr()
            rec[i]['param'] = p.data_ptr()
        host = self._host_ring[self._ring_pos]
        self._ring_pos = (self._ring_pos + 1) % len(self._host_ring)
        host.numpy()[:] = rec.view(np.uint8).reshape(-1)
        self._table.copy_(host, non_blocking=True)

    # -- public -------------------------------------------------------------------
    def grads(self) -> List[torch.Tensor]:
        out = []
        for p in self.params:
            if p.grad is None:
                raise RuntimeError('FusedAdam.step: a parameter has no gradient')
            out.append(p.grad)
        return out

    def add_sqnorm(self, accum: torch.Tensor, grads: Optional[Sequence[torch.Tensor]] = None,
                   skip: Optional[Sequence[bool]] = None) -> None:
        """Add this group's weighted squared gradient norm to the fp32 scalar tensor ``accum[0]``.

        ``skip[i]`` leaves tensor ``i`` out (its norm is already known from elsewhere)."""
        if not self.params:
            return
        grads = self.grads() if grads is None else grads
        if self.device.type == 'cuda':
            self._upload_table(grads)
            self._table_fresh = True
            blocks = self._blocks
            if skip is not None and any(skip):
                key = tuple(bool(s) for s in skip)
                if getattr(self, '_skip_key', None) != key:       # the same tensors every step: built once
                    host = self._blocks.cpu()
                    keep = ~torch.tensor(key, dtype=torch.bool)[host[:, 0].long()]
                    self._skip_key, self._skip_blocks = key, host[keep].contiguous().to(self.device)
                blocks = self._skip_blocks
            if blocks.shape[0]:
                ext().grad_sqnorm(self._table, blocks, _CHUNK, _CODES[grads[0].dtype], accum)
        else:
            for i, (g, w) in enumerate(zip(grads, self.norm_weights)):
                if skip is None or not skip[i]:
                    accum[0] += w * g.float().square().sum()

    def step(self, grad_scale: Optional[torch.Tensor] = None, grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        """One update.  ``grad_scale`` is an optional fp32 device scalar multiplied into every gradient."""
        if not self.params:
            return
        grads = self.grads() if grads is None else grads
        self.begin_step(grads)
        self.step_range(0, len(self.params), grad_scale, grads)

    def begin_step(self, grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        """Advance the step counter (bias corrections) and publish the gradient addresses.

        Followed by :meth:`step_range` calls that together cover every tensor once; the ranges
        may be launched on another stream (the table upload happens here, on the current one).
        """
        if not self.params:
            return
        self.step_count += 1
        if self.device.type == 'cuda':
            if not getattr(self, '_table_fresh', False):
                self._upload_table(self.grads() if grads is None else grads)
            self._table_fresh = False

    def step_range(self, lo: int, hi: int, grad_scale: Optional[torch.Tensor] = None,
                   grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        """Update tensors ``lo .. hi-1`` (after :meth:`begin_step`)."""
        if not self.params or hi <= lo:
            return
        grads = self.grads() if grads is None else grads
        b1, b2 = self.betas
        bias1 = 1.0 - b1**self.step_count
        bias2 = 1.0 - b2**self.step_count
        if self.device.type == 'cuda':
            blocks = self._blocks[self._block_start[lo]:self._block_start[hi]]
            ext().adam_step(self._table, blocks, _CHUNK, _CODES[self.dtype], _CODES[grads[0].dtype], self.lr, b1,
                            b2, self.eps, self.weight_decay, bias1, bias2, grad_scale, self.hyper)
            return
        scale = float(grad_scale[0]) if grad_scale is not None else 1.0
        for p, g, off in list(zip(self.params, grads, self.offsets))[lo:hi]:
            n = p.numel()
            w, m, v = (t[off:off + n] for t in (self.master, self.exp_avg, self.exp_avg_sq))
            gf = g.detach().reshape(-1).float() * scale
            m.mul_(b1).add_(gf, alpha=1 - b1)
            v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
            denom = (v / bias2).sqrt_().add_(self.eps)
            w.sub_(self.lr * ((m / bias1) / denom + self.weight_decay * w))
            p.data.copy_(w.view_as(p))

    def resync_master(self):
        """Take the fp32 master weights from the parameters again (after the model was loaded from a
        checkpoint that carries no optimizer state)."""
        for p, off in zip(self.params, self.offsets):
            self.master[off:off + p.numel()].copy_(p.detach().reshape(-1))

    def state_dict(self):
        return {'step': self.step_count, 'master': self.master, 'exp_avg': self.exp_avg,
                'exp_avg_sq': self.exp_avg_sq, 'lr': self.lr}

    def load_state_dict(self, state):
        self.step_count = int(state['step'])
        self.lr = state.get('lr', self.lr)
        if not self.params:
            return
        for name in ('master', 'exp_avg', 'exp_avg_sq'):
            getattr(self, name).copy_(state[name])
        for p, off in zip(self.params, self.offsets):
            p.data.copy_(self.master[off:off + p.numel()].view_as(p))


class Adafactor:
    """Adafactor (Shazeer & Stern, 2018) with fp32 master weights, for the reference's 760M recipe
    (``--optimizer adafactor``, exp/dmoe/dmoe_760m_8gpu.sh:70).

    Tensors with two or more dimensions keep one row statistic and one column statistic of the
    squared gradient over their last two dimensions instead of a full second moment; vectors keep
    the full moment.  The step size is the external learning rate (no relative step, no parameter
    scaling), the update is clipped to unit RMS and there is no first moment, which is how an
    absolute-lr trainer with its own schedule uses the method.  The interface is the one
    :class:`FusedAdam` offers the trainer.
    """

    def __init__(self, params: Iterable[torch.Tensor], lr: float = 1e-3, decay_rate: float = 0.8,
                 eps: float = 1e-30, clip_threshold: float = 1.0, weight_decay: float = 0.0,
                 norm_weights: Optional[Sequence[float]] = None, **_unused):
        self.params: List[torch.Tensor] = [p for p in params]
        self.lr, self.decay_rate, self.eps, self.clip_threshold = lr, decay_rate, eps, clip_threshold
        self.weight_decay = weight_decay
        self.step_count = 0
        self.norm_weights = list(norm_weights) if norm_weights is not None else [1.0] * len(self.params)
        self.device = self.params[0].device if self.params else torch.device('cpu')
        self.master = [p.detach().float().clone() for p in self.params]
        self.row, self.col, self.full = [], [], []
        for p in self.params:
            if p.dim() >= 2:
                self.row.append(torch.zeros(p.shape[:-1], dtype=torch.float32, device=p.device))
                self.col.append(torch.zeros(p.shape[:-2] + p.shape[-1:], dtype=torch.float32, device=p.device))
                self.full.append(None)
            else:
                self.row.append(None)
                self.col.append(None)
                self.full.append(torch.zeros_like(p, dtype=torch.float32))

    def grads(self) -> List[torch.Tensor]:
        out = []
        for p in self.params:
            if p.grad is None:
                raise RuntimeError('Adafactor.step: a parameter has no gradient')
            out.append(p.grad)
        return out

    def add_sqnorm(self, accum: torch.Tensor, grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        grads = self.grads() if grads is None else grads
        for g, w in zip(grads, self.norm_weights):
            accum[0] += w * g.float().square().sum()

    def begin_step(self, grads=None) -> None:
        self.step_count += 1

    def step(self, grad_scale: Optional[torch.Tensor] = None, grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        if not self.params:
            return
        self.begin_step()
        self.step_range(0, len(self.params), grad_scale, grads)

    def step_range(self, lo: int, hi: int, grad_scale: Optional[torch.Tensor] = None,
                   grads: Optional[Sequence[torch.Tensor]] = None) -> None:
        grads = self.grads() if grads is None else grads
        beta2 = 1.0 - float(self.step_count)**(-self.decay_rate)
        for i in range(lo, hi):
            p, w = self.params[i], self.master[i]
            g = grads[i].detach().float()
            if grad_scale is not None:
                g = g * grad_scale[0]
            sq = g * g + self.eps
            if self.full[i] is None:
                row, col = self.row[i], self.col[i]
                row.mul_(beta2).add_(sq.mean(dim=-1), alpha=1.0 - beta2)
                col.mul_(beta2).add_(sq.mean(dim=-2), alpha=1.0 - beta2)
                # v ~ row x col / mean(row): the rank-one reconstruction of the second moment.
                r = (row / row.mean(dim=-1, keepdim=True)).rsqrt_().unsqueeze(-1)
                c = col.rsqrt().unsqueeze(-2)
                update = g * r * c
            else:
                v = self.full[i]
                v.mul_(beta2).add_(sq, alpha=1.0 - beta2)
                update = g * v.rsqrt()
            rms = update.square().mean().sqrt()
            update = update / torch.clamp(rms / self.clip_threshold, min=1.0)
            if self.weight_decay:
                w.mul_(1.0 - self.lr * self.weight_decay)
            w.add_(update, alpha=-self.lr)
            p.data.copy_(w.view_as(p))

    def resync_master(self):
        """Take the fp32 master weights from the parameters again."""
        for p, w in zip(self.params, self.master):
            w.copy_(p.detach().reshape(w.shape))

    def state_dict(self):
        return {'step': self.step_count, 'lr': self.lr, 'master': self.master, 'row': self.row, 'col': self.col,
                'full': self.full}

    def load_state_dict(self, state):
        self.step_count = int(state['step'])
        self.lr = state.get('lr', self.lr)
        for name in ('master', 'row', 'col', 'full'):
            for dst, src in zip(getattr(self, name), state[name]):
                if dst is not None:
                    dst.copy_(src)
        for p, w in zip(self.params, self.master):
            p.data.copy_(w.view_as(p))


class DynamicLossScaler:
    """Loss scaling for fp16 training: the loss is multiplied by ``scale`` before backward and the
    gradients divided by it inside the optimizer's gradient coefficient.

    A step whose gradient norm is not finite is skipped and halves the scale (after ``hysteresis``
    such steps in a row); ``growth_interval`` clean steps in a row double it.  These are the rules of
    the mixed-precision trainer the reference's fp16 recipes run under (``--fp16`` in
    exp/moe/moe_125m_8gpu.sh and exp/dmoe/dmoe_760m_8gpu.sh; ``Arguments.fp16`` defaults to true,
    megablocks/layers/arguments.py:53).
    """

    def __init__(self, init_scale: float = 2.0**16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 1000, hysteresis: int = 2, min_scale: float = 1.0):
        self.scale = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.hysteresis, self.min_scale = growth_interval, hysteresis, min_scale
        self._good_steps = 0
        self._bad_budget = hysteresis
        self.skipped_steps = 0

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self.skipped_steps += 1
            self._good_steps = 0
            self._bad_budget -= 1
            if self._bad_budget <= 0:
                self.scale = max(self.scale * self.backoff_factor, self.min_scale)
                self._bad_budget = self.hysteresis
            return
        self._good_steps += 1
        if self._good_steps >= self.growth_interval:
            self.scale *= self.growth_factor
            self._good_steps = 0
            self._bad_budget = self.hysteresis

    def state_dict(self):
        return {'scale': self.scale, 'good_steps': self._good_steps, 'bad_budget': self._bad_budget,
                'skipped_steps': self.skipped_steps}

    def load_state_dict(self, state):
        self.scale = float(state['scale'])
        self._good_steps = int(state['good_steps'])
        self._bad_budget = int(state['bad_budget'])
        self.skipped_steps = int(state.get('skipped_steps', 0))


def clip_coefficient(sqnorm: torch.Tensor, max_norm: float, extra_scale: float = 1.0) -> torch.Tensor:
    """``[coeff, norm]`` on the device of ``sqnorm``: ``coeff = min(1, max_norm / norm) * extra_scale``."""
    out = torch.empty(2, dtype=torch.float32, device=sqnorm.device)
    if sqnorm.is_cuda:
        ext().clip_coeff(sqnorm, float(max_norm), float(extra_scale), out)
        return out
    norm = float(sqnorm[0].sqrt())
    coeff = min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0
    if not math.isfinite(norm):
        coeff = 0.0
    out[0], out[1] = coeff * extra_scale, norm
    return out


def cosine_lr(step: int, total_steps: int, peak: float, floor: float, warmup_fraction: float = 0.01) -> float:
    """Linear warm-up then cosine decay (the schedule of the reference's experiment scripts)."""
    warm = max(1, int(total_steps * warmup_fraction))
    if step < warm:
        return peak * (step + 1) / warm
    frac = min(1.0, (step - warm) / max(1, total_steps - warm))
    return floor + 0.5 * (peak - floor) * (1.0 + math.cos(math.pi * frac))
