"""Data-parallel gradient reduction by this library's peer-memory kernel, on 2+ GPUs.

The reducer's kernel (ready flags, reduce of the own slice with peer loads, stores into every
rank's slice, done flags) is compared with an fp32 average computed from all ranks' gradients
(gathered through NCCL only to build the oracle), for plain all-reduce and for the ZeRO-1
reduce-scatter, over three steps with odd-sized tensors.  A second case trains the tiny model
for two steps with both backends and compares the replicated parameters.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else (2 if n >= 2 else 0))


def _reducer_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    from megablocks_b200.parallel.dp import FlatBuffer, GradReducer
    from megablocks_b200.utils import status
    try:
        ok = True
        for shard in (False, True):
            torch.manual_seed(0)
            # ZeRO-1 shards every bucket evenly: sizes that are multiples of world x 8 elements.
            shapes = [(1000, 64), (64,), (128, 64), (640,), (512, 64)] if shard else \
                [(1000, 48), (3, 7), (129,), (64, 64), (8 * world * 5,), (500, 33)]
            params = [torch.nn.Parameter(torch.randn(*s, device=dev).bfloat16()) for s in shapes]
            flat = FlatBuffer(params, granule=world * 8)
            red = GradReducer(flat, dist.group.WORLD, bucket_bytes=16 << 10, shard=shard, backend='peer')
            assert red.backend == 'peer' and len(red.buckets) >= 2
            for step in range(3):
                flat.zero_grad()
                gen = torch.Generator(device=dev).manual_seed(1000 * step + rank)
                for p in params:
                    p.grad.copy_(torch.randn(p.shape, device=dev, generator=gen).bfloat16())
                mine = flat.grad.clone()
                gathered = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(gathered, mine)
                want = torch.stack([g.float() for g in gathered]).mean(0)
                red.finish()                       # no hooks fired: launches every bucket, then waits
                torch.cuda.synchronize()
                status.check()
                got = flat.grad.float()
                if shard:
                    for bi in range(len(red.buckets)):
                        lo, hi = red.shard_range(bi)
                        ok &= bool(torch.allclose(got[lo:hi], want[lo:hi], rtol=1e-2, atol=1e-2))
                else:
                    ok &= bool(torch.allclose(got, want, rtol=1e-2, atol=1e-2))
                    # every rank holds the same bits
                    ref = flat.grad.clone()
                    dist.broadcast(ref, src=0)
                    ok &= bool(torch.equal(ref, flat.grad))
        with open(os.path.join(out_dir, f'd{rank}.txt'), 'w') as f:
            f.write('ok' if ok else 'mismatch')
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_peer_reducer_matches_fp32_average(tmp_path):
    world = _world()
    if world < 2:
        pytest.skip('needs at least two GPUs')
    mp.spawn(_reducer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f'd{r}.txt').read() == 'ok'


def _trainer_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    from megablocks_b200.models.transformer import MoETransformer, preset
    from megablocks_b200.train import Trainer, TrainerConfig
    from megablocks_b200.utils import status
    try:
        result = {}
        for backend in ('peer', 'nccl'):
            torch.manual_seed(0)
            cfg = preset('tiny', device=dev, expert_parallel_group=dist.group.WORLD, moe_num_experts=8)
            trainer = Trainer(MoETransformer(cfg), TrainerConfig(lr=1e-3, schedule=False, bucket_mb=1,
                                                                 dp_backend=backend, grad_accum_steps=2),
                              dp_group=dist.group.WORLD)
            gen = torch.Generator().manual_seed(10 + rank)
            for _ in range(2):
                batch = torch.randint(0, cfg.vocab_size, (4, cfg.max_seq_len + 1), generator=gen).to(dev)
                trainer.step(batch[:, :-1], batch[:, 1:])
            torch.cuda.synchronize()
            status.check()
            result[backend] = torch.cat([p.detach().float().reshape(-1) for p in trainer.dense_params]).cpu()
        torch.save(result, os.path.join(out_dir, f't{rank}.pt'))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_trainer_with_peer_reducer_matches_nccl(tmp_path):
    world = _world()
    if world < 2:
        pytest.skip('needs at least two GPUs')
    mp.spawn(_trainer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f't{r}.pt')) for r in range(world)]
    for r in range(1, world):
        assert torch.equal(res[0]['peer'], res[r]['peer'])       # replicas stay bitwise in sync
    torch.testing.assert_close(res[0]['peer'], res[0]['nccl'], rtol=2e-2, atol=2e-3)


def _graph_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    from megablocks_b200.models.transformer import MoETransformer, preset
    from megablocks_b200.train import Trainer, TrainerConfig
    from megablocks_b200.utils import status
    try:
        result = {}
        for graph in (False, True):
            torch.manual_seed(0)
            cfg = preset('tiny', device=dev, expert_parallel_group=dist.group.WORLD, moe_num_experts=8)
            trainer = Trainer(MoETransformer(cfg), TrainerConfig(lr=1e-3, min_lr=1e-4, total_steps=8, warmup_fraction=0.25,
                                                                 bucket_mb=1, dp_backend='peer', cuda_graph=graph,
                                                                 graph_warmup_steps=2),
                              dp_group=dist.group.WORLD)
            gen = torch.Generator().manual_seed(10 + rank)
            losses = []
            norm_ok = True
            for it in range(7):
                batch = torch.randint(0, cfg.vocab_size, (4, cfg.max_seq_len + 1), generator=gen).to(dev)
                losses.append(trainer.step(batch[:, :-1], batch[:, 1:]))
                if it in (0, 5):
                    # The clipping norm (taken in the GEMM epilogues for the expert weights, summed over
                    # the ranks by the peer-memory kernel) against a plain sum over the gradients:
                    # replicated tensors count once, expert shards once per rank.
                    local = sum(p.grad.float().square().sum() for p in trainer.dense_params) / world + \
                        sum(p.grad.float().square().sum() for p in trainer.expert_params)
                    dist.all_reduce(local)
                    want = float(local.sqrt())
                    norm_ok &= abs(float(trainer.last_grad_norm) - want) <= 3e-3 * want
            assert norm_ok
            torch.cuda.synchronize()
            status.check()
            recorded = trainer._graph is not None
            # Back to plain launches after the replays: the sequence numbers must still line up.
            trainer.drop_graph()
            trainer.cfg.cuda_graph = False
            batch = torch.randint(0, cfg.vocab_size, (4, cfg.max_seq_len + 1), generator=gen).to(dev)
            losses.append(trainer.step(batch[:, :-1], batch[:, 1:]))
            torch.cuda.synchronize()
            status.check()
            result[graph] = {'losses': [float(l) for l in losses], 'recorded': recorded,
                             'dense': torch.cat([p.detach().float().reshape(-1) for p in trainer.dense_params]).cpu(),
                             'expert': torch.cat([p.detach().float().reshape(-1) for p in trainer.expert_params]).cpu()}
        torch.save(result, os.path.join(out_dir, f'g{rank}.pt'))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_multi_rank_step_replayed_from_a_cuda_graph(tmp_path):
    """Expert parallelism over peer memory + the peer-memory gradient reducer, recorded once and replayed:
    the same losses and weights as the step launched kernel by kernel, on every rank."""
    world = _world()
    if world < 2:
        pytest.skip('needs at least two GPUs')
    mp.spawn(_graph_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f'g{r}.pt')) for r in range(world)]
    for r in range(world):
        assert res[r][True]['recorded'] and not res[r][False]['recorded']
        torch.testing.assert_close(torch.tensor(res[r][True]['losses']), torch.tensor(res[r][False]['losses']),
                                   rtol=2e-4, atol=2e-4)
        for part in ('dense', 'expert'):
            diff = (res[r][True][part] - res[r][False][part]).abs()
            assert float(diff.median()) <= 1e-4 and float(diff.max()) <= 2 * 8 * 1e-3 + 1e-6, (r, part)
        assert torch.equal(res[0][True]['dense'], res[r][True]['dense'])        # replicas stay bitwise in sync
