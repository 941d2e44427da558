"""``custom_fwd`` / ``custom_bwd`` as stk defines them: torch's CUDA autocast decorators."""

import functools

import torch


def custom_fwd(fwd):
    return torch.amp.custom_fwd(fwd, device_type='cuda')


def custom_bwd(bwd):
    return torch.amp.custom_bwd(bwd, device_type='cuda')
