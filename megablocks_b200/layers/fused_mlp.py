"""Hand-scheduled forward/backward of the expert MLP and GLU on grouped GEMMs.

One autograd Function covers the four dropless variants: the weights are the
2-D ``[E*f, h]`` parameters viewed as ``[E, f, h]`` and the row groups are
given by ``bins`` (the inclusive prefix sum of rows per expert - the padded
prefix sum for the block-sparse layout, where every group is a multiple of 128
rows and pad rows are zero).

Forward (MLP):  ``z = x w1^T``, ``h = act(z)`` (GEMM epilogue), ``y = h w2``.
GLU: ``z1 = x w1^T`` and ``z2 = x v1^T`` come out of ONE launch whose epilogue also forms
``h = act(z1) * z2``; in backward ``dx = dz1 w1 + dz2 v1`` is one contraction over both pairs.
Backward:       ``dz = (dy w2^T) * act'(z)`` (epilogue; it also regenerates
``h`` when it was not kept), ``dw2 = h^T dy``, ``dw1 = dz^T x``, ``dx = dz w1``.
GLU adds ``z2 = x v1^T`` with ``h = act(z1) * z2`` and the matching backward.

With ``memory_optimized`` only ``x`` and the pre-activations are kept and the
activation is recomputed in the backward epilogue, the schedule of the
reference's memory-optimised Functions (megablocks/layers/mlp.py:187-305,
397-496, glu.py:66-170) without their extra elementwise passes.

Activations the kernel does not know (any Python callable) take the unfused
route: plain grouped GEMMs around the callable, differentiated by autograd.
"""

from typing import Any, Callable, Optional

import torch

from megablocks_b200.ops import gg as G


def mlp_forward(x, w1, w2, v1, bins, act: int, keep_h: bool, wait=None, zero_tail: bool = True,
                rows_hint: int = 0, scatter=None, w1_kn: bool = False):
    """Forward GEMMs.  Returns ``(y, saved)`` where ``saved = (z1, z2, h or None)``.

    ``w1`` (and ``v1``) are ``[E, f, h]``, or ``[E, h, f]`` with ``w1_kn`` (the layout of the
    token-dropping layer's experts); ``w2`` is ``[E, f, h]``.
    """
    kw = dict(zero_tail=zero_tail, rows_hint=rows_hint)
    if v1 is not None and not w1_kn and w1.shape[1] >= 128:
        # Both weight matrices in one launch: each tile multiplies its rows of x with 128 rows of w1
        # and of v1, and the epilogue forms act(z1) * z2 from the two halves of the accumulator.
        z2, h, z1 = G.grouped_gemm(x, w1, bins, trans_b=True, epilogue=G.EPI_GLU_DUAL, act=act, b2=v1, wait=wait, **kw)
    elif v1 is not None:
        z1, _, _ = G.grouped_gemm(x, w1, bins, trans_b=not w1_kn, wait=wait, **kw)
        z2, h, _ = G.grouped_gemm(x, v1, bins, trans_b=not w1_kn, epilogue=G.EPI_GLU, act=act, aux1=z1, **kw)
    else:
        z1, h, _ = G.grouped_gemm(x, w1, bins, trans_b=not w1_kn, epilogue=G.EPI_ACT, act=act, wait=wait, **kw)
        z2 = None
    # `scatter`: the last GEMM stores its rows straight into the peers' return buffers.
    y, _, _ = G.grouped_gemm(h, w2, bins, scatter=scatter, **kw)
    return y, (z1, z2, h if keep_h else None)


def mlp_backward(dy, x, w1, w2, v1, bins, act: int, saved, needs, wait=None, zero_tail: bool = True,
                 rows_hint: int = 0, scatter=None, wgrad_scale: float = 1.0, w1_kn: bool = False):
    """Backward GEMMs.  ``needs = (dx, dw1, dw2, dv1)`` flags; returns those four (``None`` where unneeded).

    ``wgrad_scale`` multiplies the weight gradients inside their GEMMs (the expert-parallel
    gradient pre-scale of megablocks/layers/mlp.py:18-32 without its extra pass over the weights).
    """
    z1, z2, h = saved
    num_experts = w1.shape[0]
    kw = dict(zero_tail=zero_tail, rows_hint=rows_hint)
    if v1 is not None:
        dz1, dz2, h_new = G.grouped_gemm(dy, w2, bins, trans_b=True, epilogue=G.EPI_DGLU, act=act, aux1=z1,
                                         aux2=z2, want_out3=h is None, wait=wait, **kw)
    else:
        dz1, h_new, _ = G.grouped_gemm(dy, w2, bins, trans_b=True, epilogue=G.EPI_DACT, act=act, aux1=z1,
                                       want_out2=h is None, wait=wait, **kw)
        dz2 = None
    if h is None:
        h = h_new
    dx = dw1 = dw2 = dv1 = None
    if needs[2]:
        dw2, _, _ = G.grouped_gemm(h, dy, bins, trans_a=True, num_groups=num_experts, alpha=wgrad_scale,
                                   grad_norm=True)
    def wgrad(dz):      # [E, f, h] = dz^T x, or [E, h, f] = x^T dz for the [E, h, f] layout
        a, b = (x, dz) if w1_kn else (dz, x)
        return G.grouped_gemm(a, b, bins, trans_a=True, num_groups=num_experts, alpha=wgrad_scale,
                              grad_norm=True)[0]

    if needs[1]:
        dw1 = wgrad(dz1)
    if v1 is not None and needs[3]:
        dv1 = wgrad(dz2)
    if needs[0]:
        # The GEMM that produces the final dx is the last reader of the receive buffers and, with
        # `scatter`, also the one that returns the rows to their sources (the epilogue that does so
        # exists for the NN layout; callers pass no `scatter` with `w1_kn`).
        if v1 is None:
            dx, _, _ = G.grouped_gemm(dz1, w1, bins, trans_b=w1_kn, scatter=scatter, **kw)
        elif not w1_kn:
            # dx = dz1 w1 + dz2 v1 as ONE contraction over both pairs: no partial result in memory.
            dx, _, _ = G.grouped_gemm(dz1, w1, bins, a2=dz2, b2=v1, scatter=scatter, **kw)
        else:
            dx, _, _ = G.grouped_gemm(dz1, w1, bins, trans_b=w1_kn, **kw)
            dx, _, _ = G.grouped_gemm(dz2, v1, bins, trans_b=w1_kn, epilogue=G.EPI_ADD, aux1=dx, scatter=scatter,
                                      **kw)
    return dx, dw1, dw2, dv1


class _ExpertMLP(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x, w1, w2, v1, bins, act: int, memory_optimized: bool, wgrad_scale: float = 1.0):
        x = x.contiguous()
        y, (z1, z2, h) = mlp_forward(x, w1, w2, v1, bins, act, keep_h=not memory_optimized)
        saved = [x, w1, w2, bins, z1]
        if v1 is not None:
            saved += [v1, z2]
        if h is not None:
            saved.append(h)
        ctx.save_for_backward(*saved)
        ctx.glu = v1 is not None
        ctx.act = act
        ctx.keep_h = h is not None
        ctx.wgrad_scale = wgrad_scale
        return y

    @staticmethod
    def backward(ctx: Any, dy):
        saved = list(ctx.saved_tensors)
        x, w1, w2, bins, z1 = saved[:5]
        v1 = z2 = None
        if ctx.glu:
            v1, z2 = saved[5:7]
        h = saved[-1] if ctx.keep_h else None
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2],
                 ctx.glu and ctx.needs_input_grad[3])
        dx, dw1, dw2, dv1 = mlp_backward(dy.contiguous(), x, w1, w2, v1, bins, ctx.act, (z1, z2, h), needs,
                                         wgrad_scale=ctx.wgrad_scale)
        return dx, dw1, dw2, dv1, None, None, None, None


def _generic(x, w1, w2, v1, bins, activation_fn: Callable):
    """Unfused route for arbitrary activation callables (autograd does the rest)."""
    z1 = G.gmm_bins(x, w1, bins, trans_b=True)
    h = activation_fn(z1)
    if v1 is not None:
        h = h * G.gmm_bins(x, v1, bins, trans_b=True)
    return G.gmm_bins(h, w2, bins)


def expert_mlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, bins: torch.Tensor,
               activation_fn: Optional[Callable], memory_optimized: bool = False,
               v1: Optional[torch.Tensor] = None, wgrad_scale: float = 1.0) -> torch.Tensor:
    """Apply every expert's MLP (or GLU when ``v1`` is given) to its group of rows.

    ``w1``/``v1``/``w2`` are ``[E, f, h]`` views of the layer parameters; their gradients come out
    multiplied by ``wgrad_scale``.
    """
    act = G.activation_id(activation_fn)
    if act is None:
        if wgrad_scale != 1.0:
            from megablocks_b200.layers.mlp import scale_gradient
            w1, w2 = scale_gradient(w1, wgrad_scale), scale_gradient(w2, wgrad_scale)
            v1 = scale_gradient(v1, wgrad_scale) if v1 is not None else None
        return _generic(x, w1, w2, v1, bins, activation_fn)
    return _ExpertMLP.apply(x, w1, w2, v1, bins, act, memory_optimized, wgrad_scale)
