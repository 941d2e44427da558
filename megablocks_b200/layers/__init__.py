from megablocks_b200.layers.dmoe import dMoE
from megablocks_b200.layers.moe import MoE

__all__ = ['MoE', 'dMoE']
