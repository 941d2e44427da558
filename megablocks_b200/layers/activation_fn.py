"""Apply an elementwise activation to a block-sparse matrix.

Reference: megablocks/layers/activation_fn.py:10-33.  The function is applied
to the stored blocks only; the topology is carried over unchanged.  With
``return_grad_fn`` the call also returns a closure that back-propagates through
the activation (used by hand-scheduled backward passes).
"""

from typing import Callable, Union

import torch

from megablocks_b200.ops import sparse


def act_fn(x: 'sparse.Matrix', function: Callable, return_grad_fn: bool = False,
           **kwargs) -> Union['sparse.Matrix', tuple]:
    if not isinstance(x, sparse.Matrix):
        raise TypeError('act_fn expects a block-sparse Matrix')
    with torch.set_grad_enabled(torch.is_grad_enabled() or return_grad_fn):
        if return_grad_fn:
            x.data.requires_grad = True
        out = function(x.data, **kwargs)
        y = sparse.with_data(x, out)
        if return_grad_fn:
            return y, out.backward
        return y
