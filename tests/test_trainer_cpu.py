"""Trainer on CPU ranks (gloo): data-parallel reduction, ZeRO-1 and expert parallelism agree with each other.

Two ranks train the tiny dMoE transformer for three steps with expert parallelism on.
Plain data parallelism and ZeRO-1 must produce the same replicated parameters on both
ranks (bitwise across ranks, closely across modes), and the fused Adam must match
``torch.optim.Adam`` on a single process.
"""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from megablocks_b200.models.transformer import MoETransformer, preset
from megablocks_b200.optim import FusedAdam
from megablocks_b200.train import Trainer, TrainerConfig


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        result = {}
        for zero1 in (False, True):
            torch.manual_seed(0)
            cfg = preset('tiny', dtype=torch.float32, expert_parallel_group=dist.group.WORLD)
            model = MoETransformer(cfg)
            trainer = Trainer(model, TrainerConfig(lr=1e-2, schedule=False, zero1=zero1, bucket_mb=1),
                              dp_group=dist.group.WORLD)
            gen = torch.Generator().manual_seed(10 + rank)
            losses = []
            for _ in range(3):
                batch = torch.randint(0, cfg.vocab_size, (2, 33), generator=gen)
                losses.append(float(trainer.step(batch[:, :-1], batch[:, 1:])))
            result[zero1] = {'losses': losses, 'norm': float(trainer.last_grad_norm),
                             'dense': torch.cat([p.detach().reshape(-1) for p in trainer.dense_params]).clone(),
                             'expert': torch.cat([p.detach().reshape(-1) for p in trainer.expert_params]).clone()}
        torch.save(result, os.path.join(out_dir, f'r{rank}.pt'))
    finally:
        dist.destroy_process_group()


def test_dp_and_zero1_agree(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(os.path.join(tmp_path, f'r{r}.pt')) for r in range(2))
    for mode in (False, True):
        assert torch.equal(r0[mode]['dense'], r1[mode]['dense'])            # replicas stay in sync
        assert not torch.equal(r0[mode]['expert'], r1[mode]['expert'])      # different experts per rank
        assert abs(r0[mode]['norm'] - r1[mode]['norm']) < 1e-5               # one global gradient norm
    # Adam turns last-bit differences of the clip coefficient into differences of order lr * 1e-2.
    torch.testing.assert_close(r0[False]['dense'], r0[True]['dense'], rtol=1e-3, atol=5e-4)
    torch.testing.assert_close(r0[False]['expert'], r0[True]['expert'], rtol=1e-3, atol=5e-4)
    assert all(abs(a - b) < 1e-3 for a, b in zip(r0[False]['losses'], r0[True]['losses']))


def test_fused_adam_matches_torch_adam():
    torch.manual_seed(0)
    params = [torch.randn(37, 5, requires_grad=True), torch.randn(129, requires_grad=True)]
    ref = [p.detach().clone().requires_grad_(True) for p in params]
    opt = FusedAdam(params, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    ropt = torch.optim.Adam(ref, lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(4):
        for p, r in zip(params, ref):
            g = torch.randn_like(p)
            p.grad, r.grad = g.clone(), g.clone()
        opt.step()
        ropt.step()
    for p, r in zip(params, ref):
        torch.testing.assert_close(p.detach(), r.detach(), rtol=1e-5, atol=1e-6)
