"""Lookup of the dropless expert module by ``(mlp_type, mlp_impl)``.

Reference: megablocks/layers/dmlp_registry.py:11-42.
"""

from typing import Union

from megablocks_b200.layers import glu, mlp
from megablocks_b200.layers.arguments import Arguments

MlpType = Union[mlp.SparseMLP, glu.SparseGLU]

_REGISTRY = {
    'mlp': {'grouped': mlp.GroupedMLP, 'sparse': mlp.SparseMLP},
    'glu': {'grouped': glu.GroupedGLU, 'sparse': glu.SparseGLU},
}


def get(args: Arguments) -> MlpType:
    """Instantiate the expert module selected by ``args.mlp_type`` / ``args.mlp_impl``."""
    by_impl = _REGISTRY.get(args.mlp_type)
    if by_impl is None:
        raise ValueError(f'Unsupported mlp type: {args.mlp_type}')
    cls = by_impl.get(args.mlp_impl)
    if cls is None:
        raise ValueError(f'{args.mlp_type} does not support {args.mlp_impl} backend.')
    return cls(args)
