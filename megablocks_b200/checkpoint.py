"""Checkpoints in the reference's state-dict format, sharded by expert-parallel rank, and resharding.

The reference has no checkpoint code of its own: a checkpoint is the
``state_dict()`` of its modules, with the names ``router.layer.weight``,
``experts.bias``, ``experts.mlp.{w1,w2,v1}`` (megablocks/layers/router.py:72-78,
moe.py:113-126, mlp.py:315-330, glu.py:23-30 of the reference), and under expert
parallelism every rank holds only its slice of the expert weights: rank ``r`` of a
world of ``W`` owns experts ``(r % esd) * E/esd ..`` and ffn rows
``(r // esd) * f/hsd ..`` where ``esd = min(W, E)`` and ``hsd = W // esd``
(mlp.py:73-83 of the reference).  This module

* saves / loads one file per rank plus a small JSON manifest,
* converts between expert-parallel degrees (``reshard``), relying only on that
  slicing rule, so a model trained at EP=8 can be loaded at EP=1, 2, 4 ... and
  back, for both the dropless (2-D) and the token-dropping (3-D) weight layouts,
* round-trips the optimizer state of :class:`megablocks_b200.train.Trainer`, also across
  expert-parallel degrees (fused Adam: per-parameter state resharded like the weights).
"""

import json
import os
import re
from typing import Dict, List

import torch

_EXPERT_KEY = re.compile(r'(^|\.)experts\.mlp\.(w1|w2|v1)$')


def is_expert_key(name: str) -> bool:
    return _EXPERT_KEY.search(name) is not None


def _degrees(world: int, num_experts: int):
    esd = min(world, num_experts)
    if num_experts % esd or world % esd:
        raise ValueError(f'cannot shard {num_experts} experts over {world} ranks')
    return esd, world // esd


def _to_full(shards: List[torch.Tensor], num_experts: int, key: str) -> torch.Tensor:
    """Reassemble ``[E, ffn, hidden]`` from per-rank shards (any source layout)."""
    world = len(shards)
    esd, hsd = _degrees(world, num_experts)
    epr = num_experts // esd
    pieces = []
    for t in shards:
        if t.dim() == 2:                       # dropless: [epr * f_local, h]
            t = t.view(epr, -1, t.shape[-1])
        elif key.endswith('w1'):               # dropping MoE w1: [epr, h, f_local]
            t = t.transpose(1, 2)
        pieces.append(t)
    rows = [torch.cat([pieces[row * esd + er] for er in range(esd)], dim=0) for row in range(hsd)]
    return torch.cat(rows, dim=1)              # [E, f, h]


def _from_full(full: torch.Tensor, world: int, rank: int, like: torch.Tensor, key: str) -> torch.Tensor:
    num_experts, ffn = full.shape[0], full.shape[1]
    esd, hsd = _degrees(world, num_experts)
    epr, rows = num_experts // esd, ffn // hsd
    e0, r0 = (rank % esd) * epr, (rank // esd) * rows
    piece = full[e0:e0 + epr, r0:r0 + rows]
    if like.dim() == 2:
        return piece.reshape(-1, full.shape[-1]).contiguous()
    if key.endswith('w1'):
        return piece.transpose(1, 2).contiguous()
    return piece.contiguous()


def reshard(shards: List[Dict[str, torch.Tensor]], new_world: int, num_experts: int) -> List[Dict[str, torch.Tensor]]:
    """Convert the per-rank model state dicts of one expert-parallel degree into another.

    Non-expert entries are replicated (taken from rank 0); expert weights are
    reassembled and re-sliced.
    """
    out: List[Dict[str, torch.Tensor]] = [dict() for _ in range(new_world)]
    for key, value in shards[0].items():
        if is_expert_key(key):
            full = _to_full([s[key] for s in shards], num_experts, key)
            for r in range(new_world):
                out[r][key] = _from_full(full, new_world, r, value, key)
        else:
            for r in range(new_world):
                out[r][key] = value.clone()
    return out


_ADAM_PARTS = ('master', 'exp_avg', 'exp_avg_sq')


def _named_opt_state(shard: Dict) -> Dict[str, Dict[str, torch.Tensor]]:
    """Cut one rank's flat Adam buffers into per-parameter tensors with the layout the trainer saved."""
    named = {}
    for opt_key, entries in shard['opt_layout'].items():
        flat = shard[opt_key]
        for name, off, shape in entries:
            n = 1
            for d in shape:
                n *= d
            named[name] = {part: flat[part][off:off + n].view(shape) for part in _ADAM_PARTS}
    return named


def save(directory: str, state: Dict, rank: int, world: int, num_experts: int, step: int = 0) -> None:
    """Write this rank's shard; rank 0 also writes ``manifest.json``."""
    os.makedirs(directory, exist_ok=True)
    torch.save(state, os.path.join(directory, f'shard_{rank:05d}_of_{world:05d}.pt'))
    if rank == 0:
        with open(os.path.join(directory, 'manifest.json'), 'w') as f:
            json.dump({'world': world, 'num_experts': num_experts, 'step': step, 'format': 'megablocks_b200/1'}, f)


def manifest(directory: str) -> Dict:
    with open(os.path.join(directory, 'manifest.json')) as f:
        return json.load(f)


def load(directory: str, rank: int, world: int, map_location='cpu') -> Dict:
    """Load the model shard for ``rank`` of ``world``, resharding if the checkpoint was saved at another degree.

    At the saved degree the shard is returned as written.  At another degree the result holds the
    resharded ``'model'`` and, when the trainer's fused Adam wrote the checkpoint, ``'opt_named'``:
    fp32 master weights and both moments per parameter name, the expert weights' state resharded by
    the same slicing rule as the weights and the replicated parameters' state taken from rank 0.
    ``Trainer.load_state_dict`` accepts either form.  ZeRO-sharded or Adafactor state is not
    converted (those moments restart).
    """
    meta = manifest(directory)
    saved_world = int(meta['world'])
    if saved_world == world:
        return torch.load(os.path.join(directory, f'shard_{rank:05d}_of_{world:05d}.pt'), map_location=map_location)
    shards = [torch.load(os.path.join(directory, f'shard_{r:05d}_of_{saved_world:05d}.pt'), map_location=map_location)
              for r in range(saved_world)]
    num_experts = int(meta['num_experts'])
    models = reshard([s['model'] for s in shards], world, num_experts)
    out = {'model': models[rank], 'step': shards[0].get('step', meta.get('step', 0))}
    if all('opt_layout' in s for s in shards):
        named = [_named_opt_state(s) for s in shards]
        out['opt_named'] = {}
        for key, entry in named[0].items():
            if is_expert_key(key):
                out['opt_named'][key] = {
                    part: _from_full(_to_full([n[key][part] for n in named], num_experts, key), world, rank,
                                     entry[part], key) for part in _ADAM_PARTS}
            else:
                out['opt_named'][key] = entry
        out['opt_step'] = shards[0]['expert_opt']['step']
        if 'loss_scaler' in shards[0]:
            out['loss_scaler'] = shards[0]['loss_scaler']
    return out
