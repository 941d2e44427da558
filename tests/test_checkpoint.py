"""Checkpoint format, sharded save / load and expert-parallel resharding (CPU)."""

from functools import partial

import pytest
import torch

import megablocks_b200 as mb
from megablocks_b200 import checkpoint
from megablocks_b200.layers import mlp as mlp_mod


def _layer(cls, **kw):
    torch.manual_seed(3)
    base = dict(hidden_size=32, ffn_hidden_size=64, moe_num_experts=4, moe_top_k=2, fp16=False,
                device=torch.device('cpu'), init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))
    base.update(kw)
    return cls(mb.Arguments(**base))


def _shards_of(full_sd, world, E):
    return checkpoint.reshard([full_sd], world, E)


@pytest.mark.parametrize('cls,kw', [(mb.dMoE, dict(mlp_type='glu')), (mb.dMoE, dict(mlp_impl='sparse')),
                                    (mb.MoE, dict())])
@pytest.mark.parametrize('world', [2, 4, 8])
def test_reshard_round_trip(cls, kw, world):
    layer = _layer(cls, **kw)
    full = {k: v.clone() for k, v in layer.state_dict().items()}
    shards = _shards_of(full, world, 4)
    assert len(shards) == world
    # Every shard follows the slicing rule of the reference (experts first, then ffn rows).
    esd, hsd = min(world, 4), world // min(world, 4)
    for r, sd in enumerate(shards):
        assert set(sd) == set(full)
        assert torch.equal(sd['router.layer.weight'], full['router.layer.weight'])
        w2 = full['experts.mlp.w2'].view(4, 64, 32) if cls is mb.dMoE else full['experts.mlp.w2']
        epr, rows = 4 // esd, 64 // hsd
        want = w2[(r % esd) * epr:(r % esd + 1) * epr, (r // esd) * rows:(r // esd + 1) * rows]
        assert torch.equal(sd['experts.mlp.w2'].reshape(want.shape), want)
    back = checkpoint.reshard(shards, 1, 4)[0]
    for k in full:
        assert torch.equal(back[k], full[k]), k
    other = checkpoint.reshard(shards, 2 if world != 2 else 4, 4)
    again = checkpoint.reshard(other, 1, 4)[0]
    for k in full:
        assert torch.equal(again[k], full[k]), k


def test_save_load_and_cross_degree_load(tmp_path):
    layer = _layer(mb.dMoE)
    full = layer.state_dict()
    shards = _shards_of(full, 4, 4)
    for r, sd in enumerate(shards):
        checkpoint.save(str(tmp_path), {'model': sd, 'step': 7}, r, 4, 4, step=7)
    assert checkpoint.manifest(str(tmp_path))['world'] == 4
    same = checkpoint.load(str(tmp_path), 2, 4)
    assert torch.equal(same['model']['experts.mlp.w1'], shards[2]['experts.mlp.w1']) and same['step'] == 7
    merged = checkpoint.load(str(tmp_path), 0, 1)
    fresh = _layer(mb.dMoE)
    fresh.load_state_dict(merged['model'])
    x = torch.randn(6, 1, 32)
    torch.testing.assert_close(fresh(x)[0], layer(x)[0])


def test_slicing_rule_matches_layer_construction():
    """The reshard rule must agree with how a layer slices freshly initialised weights per rank."""
    args = mb.Arguments(hidden_size=16, ffn_hidden_size=32, moe_num_experts=4, fp16=False, device=torch.device('cpu'))
    assert mlp_mod._rank_slice(args, 4, 32) == (slice(0, 4), slice(0, 32))
    assert checkpoint.is_expert_key('blocks.3.moe.experts.mlp.v1') and not checkpoint.is_expert_key('experts.bias')


# ---------------------------------------------------------------------------------------------
# Optimizer state across expert-parallel degrees: EP=2 -> EP=1 -> EP=2 must give back every
# rank's fp32 master weights and Adam moments bit for bit, and the merged single-process
# trainer must hold the two ranks' expert state side by side.

def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _named_state(trainer):
    out = {}
    for key, entries in trainer._opt_layout().items():
        opt = getattr(trainer, key)
        for name, off, shape in entries:
            n = int(torch.tensor(shape).prod())
            out[name] = {part: getattr(opt, part)[off:off + n].clone() for part in ('master', 'exp_avg', 'exp_avg_sq')}
    return out


def _tiny_trainer(group):
    from megablocks_b200.models.transformer import MoETransformer, preset
    from megablocks_b200.train import Trainer, TrainerConfig
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32, expert_parallel_group=group)
    model = MoETransformer(cfg)
    return cfg, Trainer(model, TrainerConfig(lr=1e-2, schedule=False, bucket_mb=1), dp_group=group)


def _ep2_worker(rank, world, port, root, phase):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        cfg, trainer = _tiny_trainer(dist.group.WORLD)
        if phase == 'train':
            gen = torch.Generator().manual_seed(20 + rank)
            for _ in range(2):
                batch = torch.randint(0, cfg.vocab_size, (2, 33), generator=gen)
                trainer.step(batch[:, :-1], batch[:, 1:])
            checkpoint.save(os.path.join(root, 'ep2'), trainer.state_dict(), rank, world, cfg.moe_num_experts, step=2)
            torch.save(_named_state(trainer), os.path.join(root, f'want{rank}.pt'))
        else:
            state = checkpoint.load(os.path.join(root, 'ep1'), rank, world)
            assert 'opt_named' in state
            trainer.load_state_dict(state)
            torch.save(_named_state(trainer), os.path.join(root, f'got{rank}.pt'))
            assert trainer.step_count == 2 and trainer.expert_opt.step_count == 2
            batch = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(5 + rank))
            assert torch.isfinite(trainer.step(batch[:, :-1], batch[:, 1:]))
    finally:
        dist.destroy_process_group()


def test_optimizer_state_survives_a_change_of_expert_parallel_degree(tmp_path):
    import os
    import torch.multiprocessing as mp
    root = str(tmp_path)
    mp.spawn(_ep2_worker, args=(2, _free_port(), root, 'train'), nprocs=2, join=True)
    # EP=2 -> one process.
    cfg, single = _tiny_trainer(None)
    state = checkpoint.load(os.path.join(root, 'ep2'), 0, 1)
    single.load_state_dict(state)
    merged = _named_state(single)
    want = [torch.load(os.path.join(root, f'want{r}.pt')) for r in range(2)]
    for name, entry in merged.items():
        for part, value in entry.items():
            if checkpoint.is_expert_key(name):
                both = torch.cat([want[0][name][part], want[1][name][part]])
                assert torch.equal(value, both), (name, part)           # dropless layout: ranks stack along rows
            else:
                assert torch.equal(value, want[0][name][part]), (name, part)
    for name, p in single.model.named_parameters():                     # weights follow the master copies
        assert torch.equal(p.detach().reshape(-1), merged[name]['master'])
    assert single.expert_opt.step_count == 2 and single.dense_opt.step_count == 2
    checkpoint.save(os.path.join(root, 'ep1'), single.state_dict(), 0, 1, cfg.moe_num_experts, step=2)
    # ... and back to EP=2: every rank gets exactly what it saved.
    mp.spawn(_ep2_worker, args=(2, _free_port(), root, 'restore'), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(os.path.join(root, f'got{r}.pt'))
        assert got.keys() == want[r].keys()
        for name in got:
            for part in got[name]:
                assert torch.equal(got[name][part], want[r][name][part]), (r, name, part)


def test_weights_only_checkpoint_refreshes_the_master_copies():
    """A checkpoint without optimizer state must not let the first update start from stale fp32 masters."""
    _, donor = _tiny_trainer(None)
    _, trainer = _tiny_trainer(None)
    with torch.no_grad():
        for p in donor.model.parameters():
            p.add_(0.25)
    trainer.load_state_dict({'model': donor.model.state_dict()})
    for opt in (trainer.dense_opt, trainer.expert_opt):
        for p, off in zip(opt.params, opt.offsets):
            assert torch.equal(opt.master[off:off + p.numel()], p.detach().reshape(-1))
    want = {n: p.detach().clone() for n, p in donor.model.named_parameters()}
    batch = torch.randint(0, 512, (2, 33), generator=torch.Generator().manual_seed(1))
    trainer.step(batch[:, :-1], batch[:, 1:])
    for n, p in trainer.model.named_parameters():       # one lr=1e-2 Adam step away from the loaded weights
        assert (p.detach() - want[n]).abs().max() <= 1.5e-2
