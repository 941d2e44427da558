"""Fused peer-memory expert parallelism on 2+ GPUs against the library all-to-all route.

Each rank builds the same dMoE layer twice (identical seed): once with
``ep_fused_comm=True`` (remote stores, per-expert flags, no NCCL) and once with
``ep_fused_comm=False`` (the step-by-step all-to-all route), feeds both the same
tokens and compares outputs and every gradient.  Skipped with fewer than two GPUs.
"""

import os
import socket
from functools import partial

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


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
            args = mb.Arguments(hidden_size=256, ffn_hidden_size=512, moe_num_experts=8, moe_top_k=kw['top_k'],
                                fp16=False, bf16=True, device=dev, bias=False, moe_loss_weight=0.0,
                                mlp_type=kw['mlp_type'], mlp_impl='grouped', memory_optimized_mlp=kw['mem_opt'],
                                moe_expert_model_parallelism=True, expert_parallel_group=dist.group.WORLD,
                                ep_fused_comm=fused,
                                init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))
            layer = mb.dMoE(args)
            torch.manual_seed(100 + rank)
            x = torch.randn(kw['tokens'], 1, 256, device=dev, dtype=torch.bfloat16).requires_grad_(True)
            probe = torch.randn(kw['tokens'], 1, 256, device=dev, dtype=torch.bfloat16)
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
            results[fused] = dict(out=outs, dx=x.grad.float().cpu(),
                                  grads={n: p.grad.float().cpu() for n, p in layer.named_parameters()})
        torch.save(results, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize('kw', [
    dict(top_k=1, mlp_type='mlp', mem_opt=True, tokens=512),
    dict(top_k=2, mlp_type='mlp', mem_opt=False, tokens=300),
    dict(top_k=2, mlp_type='glu', mem_opt=True, tokens=1024),
    dict(top_k=2, mlp_type='mlp', mem_opt=True, tokens=256, checkpoint=True),   # recomputed forward
    dict(top_k=2, mlp_type='glu', mem_opt=False, tokens=640, combine='kernel'),
])
def test_fused_matches_all_to_all(kw, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip('needs at least two GPUs')
    if world == 3:
        world = 2
    mp.spawn(_worker, args=(world, _free_port(), kw, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f'rank{r}.pt'))
        fused, plain = res[True], res[False]
        for a, b in zip(fused['out'], plain['out']):
            torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(fused['dx'], plain['dx'], rtol=2e-2, atol=2e-2)
        for name in plain['grads']:
            ref = plain['grads'][name]
            torch.testing.assert_close(fused['grads'][name], ref, rtol=3e-2, atol=2e-2 * float(ref.abs().max()) + 1e-3)
