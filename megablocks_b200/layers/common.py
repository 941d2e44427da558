"""dtype and autocast helpers (reference: megablocks/layers/common.py:9-26)."""

import torch

from megablocks_b200.layers.arguments import Arguments


def dtype(args: Arguments):
    """Parameter dtype selected by the config; ``None`` means torch's default."""
    if args.fp16:
        return torch.float16
    if args.bf16:
        return torch.bfloat16
    return None


def _autocast_dtype(device_type: str):
    if device_type == 'cuda':
        return torch.get_autocast_dtype('cuda')
    return torch.get_autocast_dtype('cpu')


def cast_if_autocast_enabled(tensor: torch.Tensor) -> torch.Tensor:
    """Cast ``tensor`` to the active autocast dtype, if autocast is on for its device."""
    device_type = 'cuda' if tensor.is_cuda else 'cpu'
    if torch.is_autocast_enabled(device_type):
        return tensor.to(dtype=_autocast_dtype(device_type))
    return tensor
