"""Fused peer-memory expert parallelism on 2+ GPUs.

Two oracles.  (1) Each rank builds the same layer twice (identical seed): once with
``ep_fused_comm=True`` (remote stores, per-expert flags, no NCCL) and once with
``ep_fused_comm=False`` (the step-by-step all-to-all route), feeds both the same tokens and
compares outputs and every gradient.  (2) The same layer evaluated in ONE process in fp32 on
all ranks' tokens (no expert parallelism at all) is compared with what the fused ranks
produced: outputs, input gradients, the router gradient summed over ranks, and each rank's
slice of the expert weight gradients.  Cases cover top-1 / top-2, MLP / GLU, the block-padded
(``sparse``) layout, Zipf-skewed routing with experts that receive nothing, unequal token
counts per rank, activation checkpointing, more ranks than experts (hidden sharding) and the
token-dropping layer with a capacity limit.  The world is every visible GPU up to 8 (2, 4
or 8).  Skipped with fewer than two GPUs.
"""

import os
import socket
from functools import partial

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HIDDEN = 256


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else (2 if n >= 2 else 0))


def _layer_args(kw, device, group=None, fused=None, dtype=torch.bfloat16):
    import megablocks_b200 as mb
    return mb.Arguments(hidden_size=HIDDEN, ffn_hidden_size=kw.get('ffn', 512), moe_num_experts=kw.get('experts', 8),
                        moe_top_k=kw['top_k'], fp16=False, bf16=dtype == torch.bfloat16, device=device, bias=False,
                        moe_loss_weight=0.0, mlp_type=kw.get('mlp_type', 'mlp'), mlp_impl=kw.get('mlp_impl', 'grouped'),
                        memory_optimized_mlp=kw.get('mem_opt', False),
                        moe_capacity_factor=kw.get('capacity_factor', 1),
                        moe_expert_model_parallelism=group is not None, expert_parallel_group=group,
                        ep_fused_comm=fused, init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))


def _skew_router(layer, kw):
    """Router whose decisions cannot flip between bf16 and fp32.

    Expert e reads input feature e only (weight 1), and the inputs carry, per token, a random
    permutation of multiples of 0.5 in their first `experts` features: any two logits of a token
    are at least 0.5 apart, far more than a bf16 rounding, so the parallel bf16 run and the fp32
    single-process oracle route every token identically.  `zipf` adds a per-expert bias (multiples of
    1/8, through a constant input feature) that skews the load; the last two experts get nothing.
    """
    with torch.no_grad():
        w = layer.router.layer.weight
        experts = w.shape[0]
        w.zero_()
        w[:, :experts] = torch.eye(experts, device=w.device, dtype=w.dtype)
        if kw.get('zipf'):
            ranks = torch.arange(1, experts + 1, dtype=torch.float32, device=w.device)
            bias = -torch.round(float(kw['zipf']) * torch.log(ranks) * 3.0 * 8.0) / 8.0
            bias[experts - 2:] = -64.0                  # nobody routes to the last two experts
            w[:, experts] = bias.to(w.dtype)            # the inputs set feature `experts` to 1


def _tokens_of(rank, kw):
    return kw['tokens'] - (rank * kw.get('uneven', 0))


def _inputs(rank, kw, device, dtype):
    gen = torch.Generator().manual_seed(100 + rank)
    n = _tokens_of(rank, kw)
    experts = kw.get('experts', 8)
    x = torch.randn(n, 1, HIDDEN, generator=gen)
    perm = torch.argsort(torch.rand(n, experts, generator=gen), dim=1).float() * 0.5
    x[:, 0, :experts] = perm
    x[:, 0, experts] = 1.0
    probe = torch.randn(n, 1, HIDDEN, generator=gen)
    return x.to(dtype).to(device), probe.to(dtype).to(device)


def _worker(rank, world, port, kw, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    # Combine either inside the last expert GEMM's epilogue (default) or by the separate return kernel.
    os.environ['MB200_EP_FUSED_COMBINE'] = '0' if kw.get('combine') == 'kernel' else '1'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    import megablocks_b200 as mb
    from megablocks_b200.utils import status
    try:
        dev = torch.device('cuda', rank)
        results = {}
        for fused in (True, False):
            torch.manual_seed(0)
            layer = getattr(mb, kw.get('cls', 'dMoE'))(_layer_args(kw, dev, dist.group.WORLD, fused))
            _skew_router(layer, kw)
            x, probe = _inputs(rank, kw, dev, torch.bfloat16)
            x.requires_grad_(True)
            outs = []
            for _ in range(2):   # two steps: sequence numbers and buffer reuse
                layer.zero_grad(set_to_none=True)
                x.grad = None
                if kw.get('checkpoint'):
                    from torch.utils.checkpoint import checkpoint
                    out = checkpoint(layer, x, use_reentrant=False)
                else:
                    out = layer(x)
                (out.float() * probe.float()).sum().backward()
                outs.append(out.detach().float().cpu())
            torch.cuda.synchronize()
            status.check()
            if fused:
                assert layer.experts._ep_workspaces, 'the fused route was not taken'
            results[fused] = dict(out=outs, dx=x.grad.float().cpu(),
                                  grads={n: p.grad.float().cpu() for n, p in layer.named_parameters()})
        torch.save(results, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


def _single_process_oracle(world, kw):
    """The layer without expert parallelism, fp32, on every rank's tokens (its weights are the bf16-rounded
    initial weights of the parallel layer)."""
    import megablocks_b200 as mb
    torch.manual_seed(0)
    dev = torch.device('cuda', 0)
    layer = getattr(mb, kw.get('cls', 'dMoE'))(_layer_args(kw, dev, dtype=torch.bfloat16))
    _skew_router(layer, kw)
    layer = layer.float()
    layer.experts.args.bf16 = layer.experts.args.fp16 = False
    outs, dxs = [], []
    for r in range(world):
        x, probe = _inputs(r, kw, dev, torch.bfloat16)
        x = x.float().requires_grad_(True)
        out = layer(x)
        (out * probe.float()).sum().backward()
        outs.append(out.detach().cpu())
        dxs.append(x.grad.cpu())
    return layer, outs, dxs


def _close(got, want, what, rtol=3e-2, scale=2e-2):
    torch.testing.assert_close(got, want, rtol=rtol, atol=scale * float(want.abs().max()) + 1e-3, msg=lambda m: f'{what}: {m}')


CASES = [
    dict(top_k=1, mem_opt=True, tokens=512),
    dict(top_k=2, tokens=300),
    dict(top_k=2, mlp_type='glu', mem_opt=True, tokens=1024),
    dict(top_k=2, mem_opt=True, tokens=256, checkpoint=True),            # recomputed forward
    dict(top_k=2, mlp_type='glu', tokens=640, combine='kernel'),
    dict(top_k=2, mlp_impl='sparse', tokens=384),                          # block-padded layout under EP
    dict(top_k=2, tokens=512, zipf=1.1, experts=16),                       # skewed load, two idle experts
    dict(top_k=1, tokens=320, uneven=32),                                  # ranks hold different token counts
    dict(top_k=1, tokens=256, experts=1, ffn=1024),                       # more ranks than experts: hidden sharding
    dict(top_k=1, tokens=512, cls='MoE', capacity_factor=1, zipf=1.1, experts=8),   # token dropping, overflowing experts
    dict(top_k=2, tokens=256, cls='MoE', capacity_factor=2),
]


@pytest.mark.gpu
@pytest.mark.parametrize('kw', CASES)
def test_fused_route(kw, tmp_path):
    world = _world()
    if world < 2:
        pytest.skip('needs at least two GPUs')
    if kw.get('experts', 8) > 1 and kw.get('experts', 8) % world:
        pytest.skip('experts do not divide over this many GPUs')
    mp.spawn(_worker, args=(world, _free_port(), kw, str(tmp_path)), nprocs=world, join=True)
    results = [torch.load(os.path.join(tmp_path, f'rank{r}.pt')) for r in range(world)]
    # (1) fused route against the all-to-all route of the same process.
    for r, res in enumerate(results):
        fused, plain = res[True], res[False]
        for a, b in zip(fused['out'], plain['out']):
            torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(fused['dx'], plain['dx'], rtol=2e-2, atol=2e-2)
        for name in plain['grads']:
            _close(fused['grads'][name], plain['grads'][name], f'rank {r} {name}')
    # (2) fused route against the fp32 single-process layer.
    if kw.get('cls') == 'MoE':
        return      # capacity-limited dropping depends on the world (which rows arrive first): oracle (1) only
    layer, outs, dxs = _single_process_oracle(world, kw)
    experts = kw.get('experts', 8)
    esd = min(world, experts)
    hsd, epr = world // esd, experts // esd
    for r, res in enumerate(results):
        _close(res[True]['out'][-1], outs[r], f'rank {r} output')
        _close(res[True]['dx'], dxs[r], f'rank {r} dx')
    total = sum(res[True]['grads']['router.layer.weight'] for res in results)
    _close(total, layer.router.layer.weight.grad.cpu(), 'router gradient', rtol=5e-2, scale=3e-2)
    names = ('w1', 'w2') + (('v1',) if kw.get('mlp_type') == 'glu' else ())
    for name in names:
        full = getattr(layer.experts.mlp, name).grad.cpu().view(experts, -1, HIDDEN)
        f_local = full.shape[1] // hsd
        for r, res in enumerate(results):
            e0, r0 = (r % esd) * epr, (r // esd) * f_local
            want = full[e0:e0 + epr, r0:r0 + f_local] / world
            _close(res[True]['grads'][f'experts.mlp.{name}'].reshape(want.shape), want, f'rank {r} {name}',
                   rtol=5e-2, scale=3e-2)
