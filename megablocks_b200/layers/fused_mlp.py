"""Hand-scheduled forward/backward of the expert MLP and GLU on grouped GEMMs.

One autograd Function covers the four dropless variants: the weights are the
2-D ``[E*f, h]`` parameters viewed as ``[E, f, h]`` and the row groups are
given by ``bins`` (the inclusive prefix sum of rows per expert - the padded
prefix sum for the block-sparse layout, where every group is a multiple of 128
rows and pad rows are zero).

Forward (MLP):  ``z = x w1^T``, ``h = act(z)`` (GEMM epilogue), ``y = h w2``.
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


class _ExpertMLP(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, x, w1, w2, v1, bins, act: int, memory_optimized: bool):
        x = x.contiguous()
        glu = v1 is not None
        if glu:
            z1, _, _ = G.grouped_gemm(x, w1, bins, trans_b=True)
            z2, h, _ = G.grouped_gemm(x, v1, bins, trans_b=True, epilogue=G.EPI_GLU, act=act, aux1=z1)
        else:
            z1, h, _ = G.grouped_gemm(x, w1, bins, trans_b=True, epilogue=G.EPI_ACT, act=act)
            z2 = None
        y, _, _ = G.grouped_gemm(h, w2, bins)
        saved = [x, w1, w2, bins, z1]
        if glu:
            saved += [v1, z2]
        if not memory_optimized:
            saved.append(h)
        ctx.save_for_backward(*saved)
        ctx.glu = glu
        ctx.act = act
        ctx.keep_h = not memory_optimized
        return y

    @staticmethod
    def backward(ctx: Any, dy):
        dy = dy.contiguous()
        saved = list(ctx.saved_tensors)
        x, w1, w2, bins, z1 = saved[:5]
        v1 = z2 = None
        if ctx.glu:
            v1, z2 = saved[5:7]
        h = saved[-1] if ctx.keep_h else None
        num_experts = w1.shape[0]

        if ctx.glu:
            dz1, dz2, h_new = G.grouped_gemm(dy, w2, bins, trans_b=True, epilogue=G.EPI_DGLU, act=ctx.act,
                                             aux1=z1, aux2=z2, want_out3=h is None)
        else:
            dz1, h_new, _ = G.grouped_gemm(dy, w2, bins, trans_b=True, epilogue=G.EPI_DACT, act=ctx.act,
                                           aux1=z1, want_out2=h is None)
            dz2 = None
        if h is None:
            h = h_new

        dw1 = dw2 = dv1 = dx = None
        if ctx.needs_input_grad[2]:
            dw2, _, _ = G.grouped_gemm(h, dy, bins, trans_a=True, num_groups=num_experts)
        if ctx.needs_input_grad[1]:
            dw1, _, _ = G.grouped_gemm(dz1, x, bins, trans_a=True, num_groups=num_experts)
        if ctx.glu and ctx.needs_input_grad[3]:
            dv1, _, _ = G.grouped_gemm(dz2, x, bins, trans_a=True, num_groups=num_experts)
        if ctx.needs_input_grad[0]:
            dx, _, _ = G.grouped_gemm(dz1, w1, bins)
            if ctx.glu:
                dx, _, _ = G.grouped_gemm(dz2, v1, bins, epilogue=G.EPI_ADD, aux1=dx)
        return dx, dw1, dw2, dv1, None, None, None


def _generic(x, w1, w2, v1, bins, activation_fn: Callable):
    """Unfused route for arbitrary activation callables (autograd does the rest)."""
    z1 = G.gmm_bins(x, w1, bins, trans_b=True)
    h = activation_fn(z1)
    if v1 is not None:
        h = h * G.gmm_bins(x, v1, bins, trans_b=True)
    return G.gmm_bins(h, w2, bins)


def expert_mlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, bins: torch.Tensor,
               activation_fn: Optional[Callable], memory_optimized: bool = False,
               v1: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Apply every expert's MLP (or GLU when ``v1`` is given) to its group of rows.

    ``w1``/``v1``/``w2`` are ``[E, f, h]`` views of the layer parameters.
    """
    act = G.activation_id(activation_fn)
    if act is None:
        return _generic(x, w1, w2, v1, bins, activation_fn)
    return _ExpertMLP.apply(x, w1, w2, v1, bins, act, memory_optimized)
