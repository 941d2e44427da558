"""Route plan: everything the permutation and the expert GEMMs need, in one call.

Given the flattened expert choice of every routed copy, produce

* ``indices``   copy id at each expert-sorted position (stable order),
* ``bin_ids``   expert of each sorted position,
* ``bins``      inclusive prefix sum of copies per expert,
* ``padded_bins`` the same after rounding each expert up to ``block`` rows,
* ``tokens_per_expert``.

The reference builds these from separate sort / histogram / round_up / cumsum
ops (megablocks/layers/moe.py:152-183, dmoe.py:131-154).  Here a CUDA input
runs a stable counting sort whose histogram and scans fall out of the same
passes (``csrc/metadata.cu``); a CPU input composes the individual ops.
"""

from typing import Tuple

import torch

from megablocks_b200._ext import ext
from megablocks_b200.ops import metadata


def route_plan(top_experts: torch.Tensor, num_experts: int,
               block: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    if top_experts.dim() != 1:
        raise ValueError('route_plan expects the flattened [tokens * top_k] expert ids')
    if top_experts.is_cuda:
        return tuple(ext().route_plan(top_experts.contiguous(), int(num_experts), int(block)))
    experts = top_experts.to(torch.int32)
    end_bit = max((num_experts - 1).bit_length(), 1)
    bin_ids, indices = metadata.sort(experts, end_bit)
    tokens_per_expert = metadata.histogram(experts, num_experts)
    bins = torch.cumsum(tokens_per_expert, 0, dtype=torch.int32)
    padded = metadata.round_up(tokens_per_expert, block)
    padded_bins = torch.cumsum(padded, 0, dtype=torch.int32)
    return indices, bin_ids, bins, padded_bins, tokens_per_expert
