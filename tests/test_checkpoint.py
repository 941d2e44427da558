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
