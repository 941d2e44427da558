"""Expert parallelism on CPU ranks (gloo): the distributed layer must equal the single-process layer.

The reference has no test of its expert-parallel path at all; these run the library
all-to-all route at world size 2 and 4 (experts sharded) and at world 4 with 2 experts
(experts *and* ffn rows sharded: "hidden sharding"), forward and backward, against the
same layer evaluated in one process on the concatenated batch.
"""

import os
import socket
from functools import partial

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import megablocks_b200 as mb


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _args(**kw):
    base = dict(hidden_size=64, ffn_hidden_size=128, moe_num_experts=4, moe_top_k=2, fp16=False, bf16=False,
                device=torch.device('cpu'), bias=False, moe_loss_weight=0.0,
                init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))
    base.update(kw)
    return base


def _worker(rank, world, port, layer_kw, cls_name, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        args = mb.Arguments(**_args(moe_expert_model_parallelism=True, expert_parallel_group=dist.group.WORLD,
                                    **layer_kw))
        layer = getattr(mb, cls_name)(args)
        torch.manual_seed(100)
        x_all = torch.randn(world, 24, 2, 64)
        x = x_all[rank].clone().requires_grad_(True)
        out = layer(x)
        probe = torch.randn(world, 24, 2, 64)[rank]
        (out * probe).sum().backward()
        grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
        torch.save({'out': out.detach(), 'dx': x.grad, 'grads': grads,
                    'tags': {n: getattr(p, 'expert_model_parallel', None) for n, p in layer.named_parameters()}},
                   os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


def _run(world, layer_kw, cls_name, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, layer_kw, cls_name, str(tmp_path)), nprocs=world, join=True)
    return [torch.load(os.path.join(tmp_path, f'rank{r}.pt')) for r in range(world)]


def _single(world, layer_kw, cls_name):
    torch.manual_seed(0)
    layer = getattr(mb, cls_name)(mb.Arguments(**_args(**layer_kw)))
    torch.manual_seed(100)
    x_all = torch.randn(world, 24, 2, 64).requires_grad_(True)
    outs = [layer(x_all[r]) for r in range(world)]
    probe = torch.randn(world, 24, 2, 64)
    sum((o * probe[r]).sum() for r, o in enumerate(outs)).backward()
    return layer, outs, x_all.grad


@pytest.mark.parametrize('world,layer_kw,cls_name', [
    (2, dict(mlp_impl='grouped'), 'dMoE'),
    (2, dict(mlp_impl='sparse', ffn_hidden_size=128), 'dMoE'),
    (2, dict(mlp_impl='grouped', mlp_type='glu'), 'dMoE'),
    (4, dict(mlp_impl='grouped', moe_top_k=1), 'dMoE'),
    (4, dict(mlp_impl='grouped', moe_num_experts=2, ffn_hidden_size=256), 'dMoE'),   # hidden sharding x2
    (2, dict(moe_capacity_factor=0), 'MoE'),
])
def test_expert_parallel_matches_single_process(world, layer_kw, cls_name, tmp_path):
    results = _run(world, layer_kw, cls_name, tmp_path)
    layer, outs, dx = _single(world, layer_kw, cls_name)
    E = layer.experts.args.moe_num_experts
    esd = min(world, E)
    hsd = world // esd
    epr = E // esd
    for r, res in enumerate(results):
        torch.testing.assert_close(res['out'], outs[r].detach(), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(res['dx'], dx[r], rtol=1e-4, atol=1e-5)
        assert res['tags']['experts.mlp.w1'] is True and res['tags']['router.layer.weight'] is None
    # Expert weight gradients: rank r holds experts (r % esd) * epr.. and ffn rows (r // esd) * f/hsd..,
    # pre-scaled by 1 / world.
    for name in ('w1', 'w2') + (('v1',) if layer_kw.get('mlp_type') == 'glu' else ()):
        full = getattr(layer.experts.mlp, name).grad
        if cls_name == 'MoE':
            full = full if name == 'w2' else full.transpose(1, 2)      # -> [E, f, h]
        else:
            full = full.view(E, -1, 64)
        f_local = full.shape[1] // hsd
        for r, res in enumerate(results):
            e0, r0 = (r % esd) * epr, (r // esd) * f_local
            want = full[e0:e0 + epr, r0:r0 + f_local] / world
            got = res['grads'][f'experts.mlp.{name}']
            if cls_name == 'MoE':
                got = got if name == 'w2' else got.transpose(1, 2)
            torch.testing.assert_close(got.reshape(want.shape), want, rtol=1e-4, atol=1e-5)
    # Router gradient: the sum over ranks equals the single-process gradient.
    total = sum(res['grads']['router.layer.weight'] for res in results)
    torch.testing.assert_close(total, layer.router.layer.weight.grad, rtol=1e-4, atol=1e-5)
