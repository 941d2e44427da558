"""Fused row-wise ops for the transformer around the MoE layers.

* :func:`cross_entropy` - mean softmax cross-entropy over ``[rows, vocab]`` logits.
  On CUDA the forward reads the 16-bit logits once (no fp32 copy) and the backward
  overwrites the logits buffer with the gradient in place, so a 3.3 GB logits tensor
  costs three passes instead of the dozen of the eager float() / log_softmax /
  nll_loss chain.  The logits tensor must not be used after the loss (it is the
  gradient afterwards).
* :func:`layer_norm` - LayerNorm whose backward reduces the weight and bias
  gradients through shared memory in the same pass that produces ``dx``.

* :func:`rms_norm` / :class:`RMSNorm` - the same kernels without centring and bias (Mixtral-style
  models), including the fused residual add.
* :func:`rope` - rotary position embedding of ``[batch, heads, seq, head_dim]`` queries / keys in
  one pass (rotation of the pairs ``(i, i + d/2)`` in fp32, no fp32 copies of the tensor).
* :func:`load_balancing_loss` - the auxiliary loss of all layers in one reduction kernel and its
  gradient in one broadcast kernel.

* :func:`linear` / :class:`Linear` - ``nn.Linear`` whose bias gradient is one column-sum kernel
  at memory bandwidth (the library route reduces the same tensor at a third of that).

All fall back to the PyTorch ops on CPU tensors.
"""

import os
from typing import Any

import torch
import torch.nn.functional as F

from megablocks_b200._ext import ext


class _CrossEntropy(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, logits: torch.Tensor, targets: torch.Tensor):
        loss, lse = ext().cross_entropy_forward(logits, targets)
        ctx.save_for_backward(logits, targets, lse)
        return loss.mean()

    @staticmethod
    def backward(ctx: Any, grad_out: torch.Tensor):
        logits, targets, lse = ctx.saved_tensors
        scale = grad_out.detach().float().reshape(1)
        ext().cross_entropy_backward_(logits, targets, lse, scale, 1.0 / logits.shape[0])
        return logits, None


class _LinearCrossEntropy(torch.autograd.Function):
    """``mean(cross_entropy(hidden @ weight^T, targets))`` with the loss and the gradient of the logits
    taken in ONE pass over the logits (they are overwritten with ``(softmax - onehot) / rows``).  The
    incoming gradient, a scalar, is then applied to the two small products of the backward pass
    instead of to the logits."""

    @staticmethod
    def forward(ctx: Any, hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor):
        logits = hidden @ weight.t()
        loss = ext().cross_entropy_fused_(logits, targets, 1.0 / logits.shape[0])
        ctx.save_for_backward(hidden, weight, logits)
        return loss.mean()

    @staticmethod
    def backward(ctx: Any, grad_out: torch.Tensor):
        hidden, weight, dlogits = ctx.saved_tensors
        scale = grad_out.detach().float()       # a 0-dim fp32 tensor: multiplies in fp32, result in the tensor's type
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh = (dlogits @ weight).mul_(scale)
        if ctx.needs_input_grad[1]:
            dw = (dlogits.t() @ hidden).mul_(scale)
        return dh, dw, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross entropy of ``hidden[rows, h] @ weight[vocab, h]^T`` against ``targets[rows]``: the
    language-model head and its loss.  On CUDA the logits are written once and read once."""
    # Not for fp16: there the loss scale has to reach the logit gradient before it is rounded (the
    # unscaled (softmax - onehot) / rows underflows), and the scale is only known in backward.
    if (hidden.is_cuda and hidden.dtype in (torch.bfloat16, torch.float32) and hidden.dim() == 2
            and weight.dtype == hidden.dtype and os.environ.get('MB200_FUSED_LM_LOSS', '1') != '0'):
        return _LinearCrossEntropy.apply(hidden.contiguous(), weight, targets.contiguous())
    return cross_entropy(F.linear(hidden, weight), targets)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross entropy of ``logits[rows, vocab]`` against ``targets[rows]`` (int64)."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float16, torch.float32) and logits.is_contiguous():
        return _CrossEntropy.apply(logits, targets.contiguous())
    return F.cross_entropy(logits.float(), targets)


class _LayerNorm(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        y, mean, rstd, _ = ext().layernorm_forward(x2, weight, bias, eps, None, None)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor):
        x2, weight, mean, rstd = ctx.saved_tensors
        dx, dw, db = ext().layernorm_backward(dy.reshape(x2.shape).contiguous(), x2, weight, mean, rstd, None, False)
        return dx.view(ctx.shape), dw, db, None


class _AddLayerNorm(torch.autograd.Function):
    """``s = a + b [+ b_bias]; y = LayerNorm(s)`` in one pass; the backward adds ``ds`` while it writes
    ``dx``.  ``b_bias`` is a per-column vector that belongs to ``b`` (the output bias of the layer that
    produced it): its add rides in the forward kernel and its gradient is one column sum of ``dx``."""

    @staticmethod
    def forward(ctx: Any, a: torch.Tensor, b: torch.Tensor, b_bias, weight: torch.Tensor, bias: torch.Tensor,
                eps: float):
        shape = a.shape
        a2 = a.reshape(-1, shape[-1]).contiguous()
        b2 = b.reshape(-1, shape[-1]).contiguous()
        y, mean, rstd, s = ext().layernorm_forward(a2, weight, bias, eps, b2, b_bias)
        ctx.save_for_backward(s, weight, mean, rstd)
        ctx.shape = shape
        ctx.bias_grad = b_bias is not None and ctx.needs_input_grad[2]
        return s.view(shape), y.view(shape)

    @staticmethod
    def backward(ctx: Any, ds, dy):
        s, weight, mean, rstd = ctx.saved_tensors
        if dy is None:
            d2 = ds.reshape(s.shape).contiguous()
            return ds, ds, (ext().column_sum(d2) if ctx.bias_grad else None), None, None, None
        dres = ds.reshape(s.shape).contiguous() if ds is not None else None
        dx, dw, db = ext().layernorm_backward(dy.reshape(s.shape).contiguous(), s, weight, mean, rstd, dres, False)
        dbias = ext().column_sum(dx) if ctx.bias_grad else None
        dx = dx.view(ctx.shape)
        return dx, dx, dbias, dw, db, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    cols = x.shape[-1]
    fused = (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and weight.dtype == x.dtype
             and bias is not None and (cols * x.element_size()) % 16 == 0 and cols <= 6144)
    if fused:
        return _LayerNorm.apply(x, weight, bias, eps)
    return F.layer_norm(x, (cols,), weight, bias, eps)


def add_layer_norm(a: torch.Tensor, b, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5, b_bias=None):
    """``(a + b, LayerNorm(a + b))``; ``b`` may be ``None``.  On CUDA the add rides in the norm's kernels.

    ``b_bias`` (optional, one value per column) is added to ``b`` in the same pass."""
    if b is None:
        return a, layer_norm(a, weight, bias, eps)
    cols = a.shape[-1]
    if b_bias is not None and not (b_bias.is_cuda and b_bias.dtype == a.dtype and b_bias.numel() == cols):
        b, b_bias = b + b_bias, None
    fused = (a.is_cuda and b.is_cuda and a.dtype == b.dtype == weight.dtype and bias is not None
             and a.shape == b.shape and a.dtype in (torch.bfloat16, torch.float16, torch.float32)
             and ext().layernorm_can_fuse(a.reshape(-1, cols)))
    if fused:
        return _AddLayerNorm.apply(a, b, b_bias, weight, bias, eps)
    s = a + b if b_bias is None else a + b + b_bias
    return s, layer_norm(s, weight, bias, eps)


class LayerNorm(torch.nn.LayerNorm):
    """``nn.LayerNorm`` (same parameters and state dict) running the fused kernels on CUDA."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return layer_norm(x, self.weight, self.bias, self.eps)

    def add_forward(self, a: torch.Tensor, b, b_bias=None):
        """``(a + b [+ b_bias], self(...))`` with the adds fused into the kernels; ``b`` may be ``None``."""
        return add_layer_norm(a, b, self.weight, self.bias, self.eps, b_bias)


class _RMSNorm(torch.autograd.Function):
    """``y = x * rsqrt(mean(x^2) + eps) * weight`` on the LayerNorm kernels (no centring, no bias)."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, weight: torch.Tensor, eps: float):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        y, mean, rstd, _ = ext().layernorm_forward(x2, weight, None, eps, None, None)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor):
        x2, weight, mean, rstd = ctx.saved_tensors
        dx, dw, _ = ext().layernorm_backward(dy.reshape(x2.shape).contiguous(), x2, weight, mean, rstd, None, True)
        return dx.view(ctx.shape), dw, None


class _AddRMSNorm(torch.autograd.Function):
    """``s = a + b; y = RMSNorm(s)`` in one pass; the backward adds ``ds`` while it writes ``dx``."""

    @staticmethod
    def forward(ctx: Any, a: torch.Tensor, b: torch.Tensor, weight: torch.Tensor, eps: float):
        shape = a.shape
        a2 = a.reshape(-1, shape[-1]).contiguous()
        b2 = b.reshape(-1, shape[-1]).contiguous()
        y, mean, rstd, s = ext().layernorm_forward(a2, weight, None, eps, b2, None)
        ctx.save_for_backward(s, weight, mean, rstd)
        ctx.shape = shape
        return s.view(shape), y.view(shape)

    @staticmethod
    def backward(ctx: Any, ds, dy):
        s, weight, mean, rstd = ctx.saved_tensors
        if dy is None:
            return ds, ds, None, None
        dres = ds.reshape(s.shape).contiguous() if ds is not None else None
        dx, dw, _ = ext().layernorm_backward(dy.reshape(s.shape).contiguous(), s, weight, mean, rstd, dres, True)
        dx = dx.view(ctx.shape)
        return dx, dx, dw, None


def _norm_kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    cols = x.shape[-1]
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32) and weight.dtype == x.dtype
            and (cols * x.element_size()) % 16 == 0 and cols <= 6144)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if _norm_kernel_ok(x, weight):
        return _RMSNorm.apply(x, weight, eps)
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def add_rms_norm(a: torch.Tensor, b, weight: torch.Tensor, eps: float = 1e-5):
    """``(a + b, RMSNorm(a + b))``; ``b`` may be ``None``.  On CUDA the add rides in the norm's kernels."""
    if b is None:
        return a, rms_norm(a, weight, eps)
    cols = a.shape[-1]
    fused = (a.is_cuda and b.is_cuda and a.dtype == b.dtype == weight.dtype and a.shape == b.shape
             and a.dtype in (torch.bfloat16, torch.float16, torch.float32)
             and ext().layernorm_can_fuse(a.reshape(-1, cols)))
    if fused:
        return _AddRMSNorm.apply(a, b, weight, eps)
    s = a + b
    return s, rms_norm(s, weight, eps)


class RMSNorm(torch.nn.Module):
    """Root-mean-square norm (weight only) running the fused kernels on CUDA."""

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight, self.eps)

    def add_forward(self, a: torch.Tensor, b, b_bias=None):
        if b is not None and b_bias is not None:
            b = b + b_bias
        return add_rms_norm(a, b, self.weight, self.eps)


class _Rope(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        ctx.save_for_backward(cos, sin)
        return ext().rope(x, cos, sin, False)

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor):
        cos, sin = ctx.saved_tensors
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        return ext().rope(dy, cos, sin, True), None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x[batch, seq, heads, dim]`` (any strides with a unit one in ``dim``) with
    fp32 tables ``cos`` / ``sin`` of shape ``[seq, dim / 2]``; pairs are ``(i, i + dim / 2)``.
    Returns a contiguous tensor."""
    d = x.shape[-1]
    elem = x.element_size()
    ok = (x.is_cuda and x.dim() == 4 and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
          and x.stride(-1) == 1 and d % (2 * (16 // elem)) == 0 and x.data_ptr() % 16 == 0
          and all((st * elem) % 16 == 0 for st in x.stride()[:3]) and cos.dtype == torch.float32)
    if ok:
        return _Rope.apply(x, cos.contiguous(), sin.contiguous())
    half = d // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:x.shape[1]].unsqueeze(1), sin[:x.shape[1]].unsqueeze(1)     # [seq, 1, dim / 2]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class _LoadBalancingLoss(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, scale: float, layers: int, *tensors):
        scores, counts = list(tensors[:layers]), list(tensors[layers:])
        ctx.scale, ctx.layers = scale, layers
        ctx.save_for_backward(*tensors)
        return ext().lbl_forward(scores, counts, scale)

    @staticmethod
    def backward(ctx: Any, gout: torch.Tensor):
        tensors = ctx.saved_tensors
        scores, counts = list(tensors[:ctx.layers]), list(tensors[ctx.layers:])
        grads = ext().lbl_backward(scores, counts, ctx.scale, gout.detach().float().reshape(1).contiguous())
        return (None, None) + tuple(grads) + (None,) * ctx.layers


def load_balancing_loss_supported(scores, counts) -> bool:
    first = scores[0]
    return (len(scores) <= 64 and all(s.is_cuda and s.is_contiguous() and s.dim() == 2 and s.shape == first.shape
                                      and s.dtype == first.dtype for s in scores)
            and first.dtype in (torch.bfloat16, torch.float16, torch.float32) and first.shape[0] > 0
            and all(c.is_cuda and c.dtype == torch.int32 and c.is_contiguous() for c in counts))


def load_balancing_loss(scores, counts, scale: float) -> torch.Tensor:
    """``scale * sum_l <counts[l], column sums of scores[l]>`` over the layers, as one fp32 scalar.

    One reduction kernel forward (fp32 accumulation, deterministic), one broadcast kernel backward.
    """
    return _LoadBalancingLoss.apply(float(scale), len(scores), *scores, *counts)


class _Linear(torch.autograd.Function):
    """``x @ w.T + b`` with library GEMMs; the bias gradient is the fused column sum."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor):
        ctx.save_for_backward(x, weight)
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = (dy2 @ weight).view(x.shape)
        if ctx.needs_input_grad[1]:
            dw = dy2.t() @ x.reshape(-1, x.shape[-1])
        if ctx.needs_input_grad[2]:
            db = ext().column_sum(dy2)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias=None) -> torch.Tensor:
    """``F.linear`` with the bias gradient computed by one bandwidth-bound kernel on CUDA."""
    fused = (bias is not None and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)
             and weight.dtype == x.dtype and bias.dtype == x.dtype and (weight.shape[0] * x.element_size()) % 16 == 0
             and not torch.is_autocast_enabled())
    if fused:
        return _Linear.apply(x, weight, bias)
    return F.linear(x, weight, bias)


class Linear(torch.nn.Linear):
    """``nn.Linear`` (same parameters and state dict) routed through :func:`linear`."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias)
