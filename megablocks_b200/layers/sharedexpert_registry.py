"""Lookup of the shared-expert module by ``mlp_type``.

Reference: megablocks/layers/sharedexpert_registry.py:9-30.
"""

from typing import Union

from megablocks_b200.layers import glu, mlp
from megablocks_b200.layers.arguments import Arguments

_REGISTRY = {'mlp': mlp.SharedMLP, 'glu': glu.SharedGLU}


def get(args: Arguments) -> Union[mlp.SharedMLP, glu.SharedGLU]:
    cls = _REGISTRY.get(args.mlp_type)
    if cls is None:
        raise ValueError(f'Unsupported mlp type: {args.mlp_type}')
    return cls(args)
