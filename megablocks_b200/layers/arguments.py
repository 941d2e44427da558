"""Configuration dataclass for the MoE / dMoE layers.

Field names and defaults follow the reference configuration object
(reference: megablocks/layers/arguments.py:22-92) so that code written against
it keeps working.  Differences, all deliberate:

* ``device`` defaults to the current CUDA device only when CUDA is present and
  to ``cpu`` otherwise, so the layer can be built on a machine without a GPU.
* ``mlp_impl='sparse'`` has no Triton dependency here (the block-sparse path is
  a native sm_100a kernel), so no Triton version check is made.
* ``mlp_impl='grouped'`` needs no external grouped-GEMM package.
"""

import dataclasses
from functools import partial
from typing import Any, Callable, Optional, Union

import torch
import torch.distributed as dist
import torch.nn.functional as F

InitFn = Union[Callable[[torch.Tensor], None], partial]

_ALLOWED_BITWIDTHS = (-1, 4, 8)

DEFAULT_ACTIVATION_FN = partial(F.gelu, approximate='tanh')

_MLP_TYPES = ('mlp', 'glu')
_MLP_IMPLS = ('sparse', 'grouped')


def _default_device() -> Union[int, torch.device]:
    if torch.cuda.is_available():
        return torch.cuda.current_device()
    return torch.device('cpu')


@dataclasses.dataclass
class Arguments:
    # Model.
    hidden_size: int = 1024
    ffn_hidden_size: int = 4096
    num_layers: int = 1
    bias: bool = True
    return_bias: bool = True
    activation_fn: Optional[Callable] = DEFAULT_ACTIVATION_FN

    # Mixture of experts.
    moe_num_experts: int = 1
    moe_top_k: int = 1
    moe_capacity_factor: int = 1
    moe_normalize_expert_weights: Optional[Union[int, float]] = None
    moe_loss_weight: float = 0.1
    moe_jitter_eps: Optional[float] = None
    moe_lbl_in_fp32: bool = False

    # Parallelism.
    moe_expert_model_parallelism: bool = False
    expert_parallel_group: Optional[dist.ProcessGroup] = None
    pipeline_model_parallel_size: int = 1
    num_layers_per_virtual_pipeline_stage: Optional[int] = None

    # Compute.
    memory_optimized_mlp: bool = False
    mlp_type: str = 'mlp'
    mlp_impl: str = 'grouped'

    # Initialisation.
    fp16: bool = True
    bf16: bool = False
    device: Union[int, torch.device] = dataclasses.field(default_factory=_default_device)
    init_method: InitFn = partial(torch.nn.init.normal_, mean=0.0, std=0.02)
    output_layer_init_method: InitFn = init_method

    # Benchmarking.
    uniform_expert_assignment: bool = False

    # Shared (always-on) expert.
    shared_expert: bool = False
    fc_cls: Any = torch.nn.Linear
    fc_kwargs: dict = dataclasses.field(default_factory=dict)
    remat_act_fn: bool = True
    shared_expert_hidden_size: Optional[int] = None
    shared_expert_weighted_sum: bool = False

    # Router z-loss.
    moe_zloss_weight: float = 0
    moe_zloss_in_fp32: bool = False

    # Extension of this library (absent from the reference): route the
    # expert-parallel exchange through the fused peer-memory kernels instead of
    # NCCL all-to-all.  ``None`` picks the fused path whenever a symmetric
    # workspace can be created for ``expert_parallel_group``.
    ep_fused_comm: Optional[bool] = None
    # Fused route only.  ``ep_max_copies``: upper bound of routed copies (tokens x top_k) any rank
    # sends in one call; the symmetric buffers are sized from it once.  ``None`` sizes them from
    # the largest first call over the group; a later call with more copies raises instead of
    # overrunning a peer's buffer.  ``ep_capacity_rows``: rows the receive buffer of a rank holds
    # (default: world x max copies, which can never overflow).  ``ep_inflight_microbatches``:
    # workspaces kept per layer, for schedules that run several forwards of a layer before the
    # first of their backwards (pipeline schedules, forward-forward-backward-backward loops).
    ep_max_copies: Optional[int] = None
    ep_capacity_rows: Optional[int] = None
    ep_inflight_microbatches: int = 1

    def __post_init__(self):
        if self.mlp_type not in _MLP_TYPES:
            raise ValueError(f'mlp_type must be one of {_MLP_TYPES}, got {self.mlp_type!r}')
        if self.mlp_impl not in _MLP_IMPLS:
            raise ValueError(f'mlp_impl must be one of {_MLP_IMPLS}, got {self.mlp_impl!r}')
        if self.shared_expert_hidden_size is None:
            self.shared_expert_hidden_size = self.ffn_hidden_size


def from_megatron(megatron_args: Any) -> Arguments:
    """Build :class:`Arguments` from any namespace that carries same-named attributes."""
    args = Arguments()
    for field in dataclasses.fields(args):
        if hasattr(megatron_args, field.name):
            setattr(args, field.name, getattr(megatron_args, field.name))
    args.__post_init__()
    return args
