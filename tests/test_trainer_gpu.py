"""Trainer on one GPU: the deferred (side-stream) expert update must not change any number."""

import pytest
import torch

from megablocks_b200.models.transformer import MoETransformer, preset
from megablocks_b200.train import Trainer, TrainerConfig


def _assert_same_training(params_a, params_b, lr: float, steps: int):
    """Two runs that differ only in the order of a few atomics.  Parameters whose true gradient is
    zero (the key part of the attention bias: softmax does not see it) carry pure rounding noise,
    and Adam's normalised update turns noise into steps of the full learning rate, so single
    elements may end up to ``2 * steps * lr`` apart; a real difference between the runs (a missed
    batch, a wrong schedule, a stale weight) moves every element and shows in the median."""
    for name in params_a:
        diff = (params_a[name] - params_b[name]).abs().flatten()
        assert float(diff.median()) <= 0.1 * lr and float(diff.max()) <= 2 * steps * lr + 1e-6, \
            (name, float(diff.median()), float(diff.max()))


def _run(overlap: bool, steps: int = 4):
    dev = torch.device('cuda', 0)
    torch.manual_seed(7)
    cfg = preset('tiny', device=dev)
    model = MoETransformer(cfg)
    trainer = Trainer(model, TrainerConfig(lr=1e-3, total_steps=100, overlap_expert_update=overlap))
    assert (trainer._update_stream is not None) == overlap
    gen = torch.Generator().manual_seed(3)
    losses = []
    for _ in range(steps):
        batch = torch.randint(0, cfg.vocab_size, (4, 65), generator=gen).to(dev)
        losses.append(trainer.step(batch[:, :-1], batch[:, 1:]))
    state = trainer.state_dict()       # flushes the side stream
    torch.cuda.synchronize()
    params = {n: p.detach().float().cpu() for n, p in model.named_parameters()}
    return [float(l) for l in losses], params, state['expert_opt']['exp_avg'].float().cpu().sum().item()


@pytest.mark.gpu
def test_deferred_expert_update_matches_inline_update():
    losses_a, params_a, m_a = _run(overlap=False)
    losses_b, params_b, m_b = _run(overlap=True)
    # Both modes order the expert parameters the same way, so the only difference left is the
    # order of a few shared-memory atomics (LayerNorm weight gradients): last-bit noise.
    torch.testing.assert_close(torch.tensor(losses_a), torch.tensor(losses_b), rtol=1e-4, atol=1e-4)
    assert abs(m_a - m_b) <= 1e-3 * max(1.0, abs(m_a))
    _assert_same_training(params_a, params_b, lr=1e-3, steps=4)
    assert losses_a[-1] < losses_a[0] + 1.0   # the run trained (no NaN, no blow-up)


def _run_graph(graph: bool, steps: int = 8):
    from megablocks_b200._ext import ext
    dev = torch.device('cuda', 0)
    torch.manual_seed(11)
    cfg = preset('tiny', device=dev)
    model = MoETransformer(cfg)
    # A short schedule, so that warm-up, peak and decay all fall inside the run.
    trainer = Trainer(model, TrainerConfig(lr=2e-3, min_lr=2e-4, total_steps=8, warmup_fraction=0.25, cuda_graph=graph,
                                           graph_warmup_steps=2))
    gen = torch.Generator().manual_seed(5)
    losses, launches = [], []
    for _ in range(steps):
        batch = torch.randint(0, cfg.vocab_size, (4, 65), generator=gen).to(dev)
        before = ext().launch_count()
        losses.append(trainer.step(batch[:, :-1], batch[:, 1:]))
        launches.append(ext().launch_count() - before)
    torch.cuda.synchronize()
    params = {n: p.detach().float().cpu() for n, p in model.named_parameters()}
    return [float(l) for l in losses], params, launches, trainer


@pytest.mark.gpu
def test_step_replayed_from_a_cuda_graph_matches_the_step_run_kernel_by_kernel():
    losses_a, params_a, launches_a, eager = _run_graph(False)
    losses_b, params_b, launches_b, graphed = _run_graph(True)
    assert eager._graph is None and graphed._graph is not None          # the third step recorded, 3..8 replayed
    # Same kernels on the same data: what differs is the order of a few atomics.  The batches
    # differ per step, so equal losses show that every replay read its own batch; equal weights
    # after a schedule of 8 different learning rates show that the replays followed the schedule.
    torch.testing.assert_close(torch.tensor(losses_a), torch.tensor(losses_b), rtol=1e-4, atol=1e-4)
    _assert_same_training(params_a, params_b, lr=2e-3, steps=8)
    assert len(set(round(l, 3) for l in losses_b)) > 4
    # Host-side counters follow the replays; a replay reports the launches it recorded.
    assert graphed.step_count == 8 and graphed.dense_opt.step_count == 8 and graphed.expert_opt.step_count == 8
    assert launches_b[-1] == launches_a[-1] > 0
    # One more step than the schedule table has rows for: the trainer goes back to plain launches.
    batch = torch.randint(0, 512, (4, 65)).to('cuda:0')
    graphed.step(batch[:, :-1], batch[:, 1:])
    extra = graphed.step(batch[:, :-1], batch[:, 1:])
    assert torch.isfinite(extra) and graphed.step_count == 10


@pytest.mark.gpu
def test_graph_is_recorded_again_after_a_checkpoint_is_loaded():
    _, _, _, trainer = _run_graph(True, steps=4)
    state = {k: (v if not isinstance(v, dict) else dict(v)) for k, v in trainer.state_dict().items()}
    state['model'] = {k: v.clone() for k, v in state['model'].items()}
    for key in ('dense_opt', 'expert_opt'):
        state[key] = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in state[key].items()}
    batch = torch.randint(0, 512, (4, 65), generator=torch.Generator().manual_seed(9)).to('cuda:0')
    want = float(trainer.step(batch[:, :-1], batch[:, 1:]))             # step 5, replayed
    trainer.load_state_dict(state)                                      # back to the state after step 4
    assert trainer._graph is None and trainer.step_count == 4
    got = float(trainer.step(batch[:, :-1], batch[:, 1:]))              # step 5 again, kernel by kernel
    assert abs(got - want) < 1e-3


@pytest.mark.gpu
def test_gradient_norm_taken_in_the_gemm_epilogues_matches_the_norm_kernel():
    """Adam hides a wrong clip coefficient (its update is scale free), so the norm itself is compared:
    the sum the weight-gradient GEMMs report, the norm kernel's, and a plain fp32 sum over ``.grad``."""
    dev = torch.device('cuda', 0)
    norms, fused_tensors = {}, {}
    for fuse in (True, False):
        torch.manual_seed(3)
        cfg = preset('tiny', device=dev)
        model = MoETransformer(cfg)
        trainer = Trainer(model, TrainerConfig(lr=1e-3, total_steps=100, fuse_grad_norm=fuse, max_grad_norm=1e9))
        batch = torch.randint(0, cfg.vocab_size, (4, 65), generator=torch.Generator().manual_seed(4)).to(dev)
        trainer.step(batch[:, :-1], batch[:, 1:])
        norms[fuse] = float(trainer.last_grad_norm)
        fused_tensors[fuse] = getattr(trainer, 'fused_norm_tensors', 0)
        plain = torch.sqrt(sum(p.grad.float().square().sum() for p in model.parameters() if p.grad is not None))
        assert abs(norms[fuse] - float(plain)) <= 2e-3 * float(plain), (fuse, norms[fuse], float(plain))
    assert fused_tensors[True] >= 2 * cfg.num_layers and fused_tensors[False] == 0
    assert abs(norms[True] - norms[False]) <= 2e-3 * norms[False]
