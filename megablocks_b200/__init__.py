"""B200-native dropless mixture-of-experts training library.

Public names match the reference package (megablocks/__init__.py:4-20).
"""

from megablocks_b200._version import __version__
from megablocks_b200.layers.arguments import Arguments
from megablocks_b200.layers.dmoe import ParallelDroplessMLP, dMoE
from megablocks_b200.layers.glu import SparseGLU
from megablocks_b200.layers.mlp import MLP, SparseMLP
from megablocks_b200.layers.moe import MoE, ParallelMLP, get_load_balancing_loss

__all__ = [
    'MoE',
    'dMoE',
    'get_load_balancing_loss',
    'ParallelMLP',
    'ParallelDroplessMLP',
    'SparseMLP',
    'MLP',
    'SparseGLU',
    'Arguments',
    '__version__',
]
