"""Expert-parallel sharding arithmetic and parameter tagging.

Reference behaviour: megablocks/layers/mpu.py:12-93.  With ``W`` ranks in the
expert-parallel group and ``E`` experts, experts are split ``min(W, E)`` ways
and, when ``W > E``, every expert's ffn dimension is further split
``W // min(W, E)`` ways ("hidden sharding").
"""

from typing import Optional

import torch
import torch.distributed as dist

from megablocks_b200.layers.arguments import Arguments


class MoeParam(torch.Tensor):
    """Typing aid: a parameter that carries ``expert_model_parallel``."""

    expert_model_parallel: bool


def is_moe_param(tensor: torch.Tensor) -> bool:
    return hasattr(tensor, 'expert_model_parallel')


def get_expert_parallel_world_size(args: Arguments) -> int:
    if not args.moe_expert_model_parallelism:
        return 1
    return dist.get_world_size(args.expert_parallel_group)


def get_expert_parallel_rank(args: Arguments) -> int:
    if not args.moe_expert_model_parallelism:
        return 0
    return dist.get_rank(args.expert_parallel_group)


def set_expert_model_parallel_attributes(tensor: torch.Tensor, is_parallel: bool) -> None:
    if hasattr(tensor, 'expert_model_parallel'):
        raise AssertionError('expert_model_parallel is already set on this tensor')
    tensor.expert_model_parallel = is_parallel


def param_is_expert_model_parallel(param: torch.Tensor) -> bool:
    return bool(getattr(param, 'expert_model_parallel', False))


def copy_expert_model_parallel_attributes(destination_tensor: torch.Tensor, source_tensor: torch.Tensor) -> None:
    if hasattr(source_tensor, 'expert_model_parallel'):
        destination_tensor.expert_model_parallel = source_tensor.expert_model_parallel


def synchronized_print(group: Optional[dist.ProcessGroup], *x) -> None:
    """Print from every rank of ``group`` in rank order."""
    me = dist.get_rank(group)
    for turn in range(dist.get_world_size(group)):
        dist.barrier(group)
        if turn == me:
            print(f'rank = {me}', *x)


def expert_sharding_degree(args: Arguments) -> int:
    world = get_expert_parallel_world_size(args)
    degree = min(world, args.moe_num_experts)
    if args.moe_num_experts % degree:
        raise ValueError(f'Cannot shard {args.moe_num_experts} experts {degree} ways.')
    return degree


def hidden_sharding_degree(args: Arguments) -> int:
    world = get_expert_parallel_world_size(args)
    esd = expert_sharding_degree(args)
    hsd = world // esd
    if args.ffn_hidden_size % hsd:
        raise ValueError(f'Cannot shard {args.ffn_hidden_size} features {hsd} ways.')
    if esd * hsd != world:
        raise ValueError(
            f"Invalid sharding. 'expert_sharding_degree' ({esd}) * hidden_sharding_degree ({hsd}) "
            f'!= world_size ({world}).')
    return hsd


def experts_per_rank(args: Arguments) -> int:
    return args.moe_num_experts // expert_sharding_degree(args)


def features_per_rank(args: Arguments) -> int:
    return args.ffn_hidden_size // hidden_sharding_degree(args)
