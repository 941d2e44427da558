"""Trainer features of the reference's recipes, on CPU: gradient accumulation, fp16 loss scaling,
Adafactor, and a two-stage pipeline (gloo ranks) that must reproduce the single-process step.
"""

import copy
import os
import sys
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from megablocks_b200.models.transformer import MoETransformer, preset
from megablocks_b200.optim import Adafactor, DynamicLossScaler
from megablocks_b200.train import Trainer, TrainerConfig


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _flat(params):
    return torch.cat([p.detach().reshape(-1) for p in params])


def test_gradient_accumulation_matches_one_large_batch():
    """Two micro-batches of 2 sequences = one batch of 4: same loss, same gradient norm, same update.

    The load-balancing loss is off: it is a product of two per-batch means and so, unlike the
    language-model loss, not additive over micro-batches.
    """
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32, moe_loss_weight=0.0)
    base = MoETransformer(cfg)
    batch = torch.randint(0, cfg.vocab_size, (4, 33))
    outs = []
    for accum in (1, 2):
        model = copy.deepcopy(base)
        trainer = Trainer(model, TrainerConfig(lr=1e-2, schedule=False, grad_accum_steps=accum))
        loss = trainer.step(batch[:, :-1], batch[:, 1:])
        outs.append((float(loss), float(trainer.last_grad_norm), _flat(model.parameters())))
    assert abs(outs[0][0] - outs[1][0]) < 1e-5
    assert abs(outs[0][1] - outs[1][1]) < 1e-4
    # Adam turns last-bit gradient differences into update differences of order lr * 1e-2.
    torch.testing.assert_close(outs[0][2], outs[1][2], rtol=1e-3, atol=5e-4)


def test_loss_scaler_rules():
    s = DynamicLossScaler(init_scale=1024.0, growth_interval=3, hysteresis=2)
    s.update(True)
    assert s.scale == 1024.0 and s.skipped_steps == 1           # first overflow is tolerated
    s.update(True)
    assert s.scale == 512.0                                      # second in a row halves the scale
    for _ in range(3):
        s.update(False)
    assert s.scale == 1024.0                                     # three clean steps double it
    restored = DynamicLossScaler()
    restored.load_state_dict(s.state_dict())
    assert restored.scale == s.scale and restored.skipped_steps == 2


def test_loss_scaling_skips_overflowed_steps_and_unscales_the_rest():
    """With scaling forced on (fp32 weights, so the arithmetic is exact) a finite step equals the
    unscaled step, and a step whose gradients overflow leaves the weights untouched."""
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32)
    base = MoETransformer(cfg)
    batch = torch.randint(0, cfg.vocab_size, (2, 33))
    plain, scaled = copy.deepcopy(base), copy.deepcopy(base)
    t_plain = Trainer(plain, TrainerConfig(lr=1e-2, schedule=False))
    t_scaled = Trainer(scaled, TrainerConfig(lr=1e-2, schedule=False, loss_scaling=True, init_loss_scale=256.0))
    t_plain.step(batch[:, :-1], batch[:, 1:])
    t_scaled.step(batch[:, :-1], batch[:, 1:])
    torch.testing.assert_close(_flat(scaled.parameters()), _flat(plain.parameters()), rtol=1e-4, atol=1e-6)
    assert abs(float(t_scaled.last_grad_norm) - float(t_plain.last_grad_norm)) < 1e-3

    before = _flat(scaled.parameters()).clone()
    t_scaled.scaler.scale = float('inf')                         # every gradient overflows
    t_scaled.step(batch[:, :-1], batch[:, 1:])
    assert torch.equal(_flat(scaled.parameters()), before)
    assert t_scaled.scaler.skipped_steps == 1 and t_scaled.step_count == 1


def test_adafactor_reduces_the_loss_and_keeps_factored_state():
    torch.manual_seed(0)
    w = torch.randn(64, 32, requires_grad=True)
    b = torch.zeros(32, requires_grad=True)
    x, y = torch.randn(256, 64), torch.randn(256, 32)
    opt = Adafactor([w, b], lr=3e-2)
    assert opt.row[0].shape == (64,) and opt.col[0].shape == (32,) and opt.full[0] is None
    assert opt.full[1].shape == (32,)
    losses = []
    for _ in range(60):
        loss = ((x @ w + b - y)**2).mean()
        losses.append(float(loss.detach()))
        w.grad, b.grad = torch.autograd.grad(loss, (w, b))
        opt.step()
    assert losses[-1] < 0.5 * losses[0]
    # Every update is clipped to unit RMS, so one step moves a weight by at most about lr.
    clone = w.detach().clone()
    w.grad, b.grad = torch.full_like(w, 1e6), torch.zeros_like(b)
    opt.step()
    assert float((w.detach() - clone).abs().max()) < 10 * 3e-2
    state = opt.state_dict()
    other = Adafactor([w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)], lr=3e-2)
    other.load_state_dict(state)
    assert other.step_count == opt.step_count and torch.equal(other.row[0], opt.row[0])


def test_trainer_runs_with_adafactor():
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32)
    model = MoETransformer(cfg)
    trainer = Trainer(model, TrainerConfig(lr=1e-2, schedule=False, optimizer='adafactor'))
    batch = torch.randint(0, cfg.vocab_size, (2, 33))
    first = float(trainer.step(batch[:, :-1], batch[:, 1:]))
    for _ in range(5):
        last = float(trainer.step(batch[:, :-1], batch[:, 1:]))
    assert last < first


# ---------------------------------------------------------------------------------------------
# pipeline: 2 stages on 2 gloo ranks vs the same weights in one process
# ---------------------------------------------------------------------------------------------
def _pipeline_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from megablocks_b200.parallel.pipeline import PipelineStage
        torch.manual_seed(0)
        full_cfg = preset('tiny', dtype=torch.float32, flavour='mixtral', num_kv_heads=2, moe_num_experts=4)
        full = MoETransformer(full_cfg)                       # same seed on both ranks: same weights
        cfg = preset('tiny', dtype=torch.float32, flavour='mixtral', num_kv_heads=2, moe_num_experts=4,
                     pipeline_stages=2, pipeline_stage=rank)
        stage_model = MoETransformer(cfg)
        # Copy this stage's slice of the full model.
        own = stage_model.state_dict()
        source = full.state_dict()
        layers_per_stage = full_cfg.num_layers // 2
        for key in own:
            src_key = key
            if key.startswith('blocks.'):
                idx = int(key.split('.')[1])
                src_key = 'blocks.%d.%s' % (idx + rank * layers_per_stage, key.split('.', 2)[2])
            own[key].copy_(source[src_key])
        assert len(stage_model.blocks) == layers_per_stage
        stage = PipelineStage(dist.group.WORLD, (2, 32, cfg.hidden_size), torch.float32, torch.device('cpu'))
        trainer = Trainer(stage_model, TrainerConfig(lr=1e-2, schedule=False, grad_accum_steps=2, max_grad_norm=1.0),
                          pipeline=stage)
        batch = torch.randint(0, cfg.vocab_size, (4, 33), generator=torch.Generator().manual_seed(3))
        loss = trainer.step(batch[:, :-1], batch[:, 1:])
        result = {'loss': float(loss), 'norm': float(trainer.last_grad_norm),
                  'params': {k: v.clone() for k, v in stage_model.state_dict().items()}}
        if rank == 0:
            ref = Trainer(full, TrainerConfig(lr=1e-2, schedule=False, grad_accum_steps=2, max_grad_norm=1.0))
            ref_loss = ref.step(batch[:, :-1], batch[:, 1:])
            result['ref'] = {'loss': float(ref_loss), 'norm': float(ref.last_grad_norm),
                             'params': {k: v.clone() for k, v in full.state_dict().items()}}
        torch.save(result, os.path.join(out_dir, f'p{rank}.pt'))
    finally:
        dist.destroy_process_group()


def test_two_stage_pipeline_matches_single_process(tmp_path):
    mp.spawn(_pipeline_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(os.path.join(tmp_path, f'p{r}.pt')) for r in range(2))
    ref = r0['ref']
    assert abs(r1['loss'] - ref['loss']) < 1e-5                  # the last stage sees the loss
    assert abs(r0['norm'] - ref['norm']) < 1e-4 and abs(r1['norm'] - ref['norm']) < 1e-4
    layers_per_stage = 1
    for rank, res in ((0, r0), (1, r1)):
        for key, value in res['params'].items():
            src_key = key
            if key.startswith('blocks.'):
                idx = int(key.split('.')[1])
                src_key = 'blocks.%d.%s' % (idx + rank * layers_per_stage, key.split('.', 2)[2])
            torch.testing.assert_close(value, ref['params'][src_key], rtol=1e-4, atol=1e-5, msg=key)


def test_pipeline_stage_checks_its_load_balancing_terms():
    """A stage must have collected num_layers / stages load-balancing terms (the reference's rule)."""
    from megablocks_b200.layers.moe import batched_load_balancing_loss, clear_load_balancing_loss
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32, pipeline_stages=2, pipeline_stage=0)
    model = MoETransformer(cfg).train()
    tokens = torch.randint(0, cfg.vocab_size, (2, 32))
    hidden, aux = model.stage_forward(tokens)
    assert aux is not None and hidden.shape == (2, 32, cfg.hidden_size)
    # Two forwards without clearing in between: twice the terms a stage may hold.
    model._run_blocks(model._embed(tokens))
    model._run_blocks(model._embed(tokens))
    with pytest.raises(ValueError, match='Expected 1 token_per_experts'):
        batched_load_balancing_loss(model.moe_args)
    clear_load_balancing_loss()


def test_run_from_host_returns_every_loss_in_order():
    """The pipelined host loop gives the same losses as one blocking call per step."""
    torch.manual_seed(0)
    cfg = preset('tiny', dtype=torch.float32)
    base = MoETransformer(cfg)
    batches = [torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(i)) for i in range(4)]
    a = Trainer(copy.deepcopy(base), TrainerConfig(lr=1e-2, schedule=False))
    b = Trainer(copy.deepcopy(base), TrainerConfig(lr=1e-2, schedule=False))
    want = [a.step_from_host(x) for x in batches]
    got = b.run_from_host(iter(batches))
    assert len(got) == 4 and all(abs(p - q) < 1e-6 for p, q in zip(want, got))
    assert b.run_from_host([]) == []


def test_fused_adam_norm_can_leave_tensors_out():
    """``add_sqnorm(skip=...)``: tensors whose norm is known from elsewhere are not summed again."""
    from megablocks_b200.optim import FusedAdam
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(5, 3)), torch.nn.Parameter(torch.randn(7)), torch.nn.Parameter(torch.randn(2, 2))]
    for p in params:
        p.grad = torch.randn_like(p)
    opt = FusedAdam(params, lr=1e-3)
    full, part = torch.zeros(1), torch.zeros(1)
    opt.add_sqnorm(full)
    opt.add_sqnorm(part, skip=[False, True, False])
    want_full = sum(float(p.grad.square().sum()) for p in params)
    want_part = want_full - float(params[1].grad.square().sum())
    assert abs(float(full) - want_full) < 1e-4 and abs(float(part) - want_part) < 1e-4


def test_grad_norm_sink_lookup_is_by_address_and_size():
    from megablocks_b200.ops.gg import GradNormSink
    sink = GradNormSink(torch.device('cpu'), slots=4)
    sink.begin()
    a, b = torch.zeros(6), torch.zeros(6)
    slot, view = sink._next()
    assert slot == 0 and view.numel() == 1
    sink._record(a, slot)
    assert sink.lookup(a) == 0 and sink.lookup(b) is None and sink.lookup(a[:3]) is None
    sink.begin()
    assert sink.lookup(a) is None and float(sink.slots.sum()) == 0.0


def test_experiment_scripts_are_valid_shell_and_use_known_flags_and_presets():
    """Every script under exp/ parses as bash, names an existing preset and passes only flags the trainer's
    command line knows."""
    import glob
    import re
    import subprocess
    from megablocks_b200.models.transformer import PRESETS
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    scripts = sorted(glob.glob(os.path.join(root, 'exp', '*', '*.sh')))
    assert len(scripts) == 17
    help_text = subprocess.run([sys.executable, '-m', 'megablocks_b200.train', '--help'], capture_output=True, text=True,
                               cwd=root, check=True).stdout
    known = set(re.findall(r'(--[a-z][a-z0-9-]*)', help_text))
    launcher = {'--nnodes', '--nproc-per-node', '--master-addr', '--master-port'}
    for path in scripts:
        assert subprocess.run(['bash', '-n', path]).returncode == 0, path
        text = open(path).read()
        command = text[text.index('python -m torch.distributed.run'):]
        preset = re.search(r'--preset (\S+)', command).group(1)
        assert preset in PRESETS, (path, preset)
        for flag in set(re.findall(r'(--[a-z][a-z0-9-]*)', command)) - launcher:
            assert flag in known, (path, flag)
