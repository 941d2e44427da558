"""Closed-form tanh-GELU and its backward (reference: megablocks/layers/gelu.py:9-43).

``gelu`` / ``gelu_backward_`` accept either a plain tensor or a block-sparse
:class:`megablocks_b200.ops.sparse.Matrix`; for a matrix they act on its value
array and keep its topology.  ``gelu_backward_`` overwrites ``grad``.
"""

import torch
import torch.nn.functional as F

from megablocks_b200.ops import sparse

_K0 = 0.79788456
_K1 = 0.035677408136300125  # 0.79788456 * 0.044715
_K2 = 0.1070322243          # 3 * 0.79788456 * 0.044715


def _gelu_backward_inplace(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    t = torch.tanh(x * (_K0 + _K1 * x * x))
    slope = 0.5 * x * ((1 - t * t) * (_K0 + _K2 * x * x)) + 0.5 * (1 + t)
    return g.mul_(slope)


def gelu_backward_(grad, x):
    if isinstance(grad, sparse.Matrix):
        if not isinstance(x, sparse.Matrix):
            raise ValueError('grad and x must both be block-sparse or both be dense')
        return sparse.with_data(grad, _gelu_backward_inplace(grad.data, x.data))
    return _gelu_backward_inplace(grad, x)


def gelu(x):
    if isinstance(x, sparse.Matrix):
        return sparse.with_data(x, F.gelu(x.data, approximate='tanh'))
    return F.gelu(x, approximate='tanh')
