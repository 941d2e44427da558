"""Public ops namespace (same names as ``megablocks.ops``) plus this library's additions."""

from megablocks_b200.ops.gg import gmm, gmm_bins, grouped_gemm
from megablocks_b200.ops.metadata import (exclusive_cumsum, histogram, inclusive_cumsum, repeat, replicate,
                                          round_up, sort, sum, topology)
from megablocks_b200.ops.permute import (binned_gather, binned_scatter, gather, padded_gather, padded_scatter,
                                         scatter)
from megablocks_b200.ops.route import route_plan
from megablocks_b200.ops.sparse import Matrix, dds, dsd, sdd

__all__ = [
    'binned_gather',
    'binned_scatter',
    'exclusive_cumsum',
    'inclusive_cumsum',
    'gather',
    'histogram',
    'padded_gather',
    'padded_scatter',
    'repeat',
    'replicate',
    'round_up',
    'scatter',
    'sort',
    'sum',
    'topology',
    # additions
    'gmm',
    'gmm_bins',
    'grouped_gemm',
    'route_plan',
    'Matrix',
    'sdd',
    'dsd',
    'dds',
]
