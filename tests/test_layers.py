"""Layer-level checks: shapes, numerics against dense per-expert loops, losses, state dicts.

Mirrors the reference layer tests (tests/layers/dmoe_test.py:17-241, moe_test.py:155-199,
glu_test.py:64-123) and adds backward numerics, which the reference only smoke-tests.
"""

from functools import partial

import pytest
import torch
import torch.nn.functional as F
from conftest import DEVICES

import megablocks_b200 as mb
from megablocks_b200.layers import moe as moe_mod
from megablocks_b200.layers import router as router_mod
from megablocks_b200.layers.arguments import from_megatron

CONFIGS = [(8, 16, 128, 1, 1), (8, 16, 128, 2, 1), (8, 16, 128, 4, 1), (8, 16, 128, 4, 2), (8, 16, 256, 8, 4),
           (2, 64, 128, 8, 2), (1, 33, 128, 5, 3)]


def _args(device, hs=128, ffn=None, ne=8, top_k=2, **kw):
    half = device == 'cuda'
    base = dict(hidden_size=hs, ffn_hidden_size=ffn or 2 * hs, moe_num_experts=ne, moe_top_k=top_k, fp16=False,
                bf16=half, device=torch.device(device), moe_capacity_factor=1, memory_optimized_mlp=False,
                init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))
    base.update(kw)
    return mb.Arguments(**base)


def _tol(device):
    return dict(rtol=3e-2, atol=3e-2) if device == 'cuda' else dict(rtol=1e-5, atol=1e-5)


def dense_oracle(layer, x, mlp_type='mlp'):
    """Per-expert dense loop in fp32: the definition of the dropless layer."""
    args = layer.experts.args
    E, k, h = args.moe_num_experts, args.moe_top_k, args.hidden_size
    xf = x.reshape(-1, h).float()
    wr = layer.router.layer.weight.float()
    scores = (xf @ wr.t()).softmax(-1)
    if x.is_cuda:
        # 16-bit scores can order a near-tie differently from fp32; take the layer's own
        # choice of experts and check everything else (weights, experts, gradients) in fp32.
        with torch.no_grad():
            e = layer.router(x)[2]
        w = scores.gather(1, e)
    else:
        w, e = torch.topk(scores, k, dim=-1)
    if args.moe_normalize_expert_weights:
        w = w / torch.norm(w, p=args.moe_normalize_expert_weights, dim=-1, keepdim=True)
    w1 = layer.experts.mlp.w1.float().view(E, -1, h)
    w2 = layer.experts.mlp.w2.float().view(E, -1, h)
    v1 = layer.experts.mlp.v1.float().view(E, -1, h) if mlp_type == 'glu' else None
    out = torch.zeros_like(xf)
    for ex in range(E):
        for s in range(k):
            sel = e[:, s] == ex
            if not sel.any():
                continue
            hid = args.activation_fn(xf[sel] @ w1[ex].t())
            if v1 is not None:
                hid = hid * (xf[sel] @ v1[ex].t())
            out[sel] += w[sel, s:s + 1] * (hid @ w2[ex])
    return out.view(x.shape), scores, e


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('bs,sl,hs,ne,top_k', CONFIGS)
@pytest.mark.parametrize('mlp_impl', ['grouped', 'sparse'])
@pytest.mark.parametrize('mlp_type', ['mlp', 'glu'])
@pytest.mark.parametrize('mem_opt', [False, True])
def test_dmoe_matches_dense_loop(device, bs, sl, hs, ne, top_k, mlp_impl, mlp_type, mem_opt):
    args = _args(device, hs=hs, ne=ne, top_k=top_k, mlp_impl=mlp_impl, mlp_type=mlp_type,
                 memory_optimized_mlp=mem_opt)
    layer = mb.dMoE(args)
    x = torch.randn(sl, bs, hs, device=device).to(layer.router.layer.weight.dtype).requires_grad_(True)
    out, bias = layer(x)
    assert out.shape == x.shape and bias.shape == (hs,)
    ref, _, _ = dense_oracle(layer, x, mlp_type)
    torch.testing.assert_close(out.float(), ref, **_tol(device))

    params = [layer.experts.mlp.w1, layer.experts.mlp.w2, layer.router.layer.weight, x]
    if mlp_type == 'glu':
        params.append(layer.experts.mlp.v1)
    probe = torch.randn_like(ref)
    got = torch.autograd.grad((out.float() * probe).sum(), params)
    want = torch.autograd.grad((ref * probe).sum(), params)
    for g, w_ in zip(got, want):
        tol = _tol(device)
        if device == 'cuda':   # 16-bit gradients carry rounding proportional to their magnitude
            tol = dict(rtol=5e-2, atol=3e-2 * float(w_.abs().max()) + 1e-3)
        torch.testing.assert_close(g.float(), w_.float(), **tol)


def test_config1_cpu_plumbing():
    """One dMoE layer, hidden 128, ffn 512, 8 experts, top-2, GELU, x[32,2,128] from seed 0: 1e-5."""
    torch.manual_seed(0)
    args = mb.Arguments(hidden_size=128, ffn_hidden_size=512, moe_num_experts=8, moe_top_k=2, fp16=False,
                        device=torch.device('cpu'))
    layer = mb.dMoE(args)
    x = torch.randn(32, 2, 128, requires_grad=True)
    out, _ = layer(x)
    ref, _, _ = dense_oracle(layer, x)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    g = torch.autograd.grad(out.square().sum(), [x, layer.experts.mlp.w1, layer.experts.mlp.w2])
    r = torch.autograd.grad(ref.square().sum(), [x, layer.experts.mlp.w1, layer.experts.mlp.w2])
    for a, b in zip(g, r):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('bs,sl,hs,ne,top_k', CONFIGS[:5])
def test_moe_capacity0_equals_dmoe(device, bs, sl, hs, ne, top_k):
    args = _args(device, hs=hs, ne=ne, top_k=top_k, moe_capacity_factor=0)
    moe = mb.MoE(args)
    dmoe = mb.dMoE(_args(device, hs=hs, ne=ne, top_k=top_k, mlp_impl='grouped'))
    with torch.no_grad():
        dmoe.router.layer.weight.copy_(moe.router.layer.weight)
        E = ne
        dmoe.experts.mlp.w1.copy_(moe.experts.mlp.w1.transpose(1, 2).reshape(-1, hs))
        dmoe.experts.mlp.w2.copy_(moe.experts.mlp.w2.reshape(-1, hs))
    x = torch.randn(sl, bs, hs, device=device).to(moe.router.layer.weight.dtype)
    a, _ = moe(x)
    b, _ = dmoe(x)
    torch.testing.assert_close(a.float(), b.float(), **_tol(device))


@pytest.mark.parametrize('device', DEVICES)
def test_moe_drops_tokens_beyond_capacity(device):
    args = _args(device, hs=128, ne=4, top_k=1, moe_capacity_factor=1, bias=False)
    layer = mb.MoE(args)
    with torch.no_grad():  # route everything to expert 0
        layer.router.layer.weight.zero_()
        layer.router.layer.weight[0].fill_(1.0)
    x = torch.rand(64, 1, 128, device=device).to(layer.router.layer.weight.dtype) + 0.5
    out = layer(x)
    kept = (out.float().abs().sum(-1) > 0).sum().item()
    assert kept == 16  # capacity = 1 * 64 / 4


@pytest.mark.parametrize('device', DEVICES)
def test_forward_return_modes_and_shared_expert(device):
    x = torch.randn(16, 2, 128, device=device)
    for bias, return_bias in [(True, True), (True, False), (False, True)]:
        layer = mb.dMoE(_args(device, bias=bias, return_bias=return_bias))
        out = layer(x.to(layer.router.layer.weight.dtype))
        if bias and return_bias:
            assert isinstance(out, tuple) and out[1] is layer.experts.bias
        else:
            assert out.shape == x.shape
    for typ in ('mlp', 'glu'):
        for weighted in (False, True):
            layer = mb.dMoE(_args(device, bias=False, shared_expert=True, mlp_type=typ,
                                  shared_expert_weighted_sum=weighted, shared_expert_hidden_size=64))
            layer.shared_expert.to(layer.router.layer.weight.dtype)
            xx = x.to(layer.router.layer.weight.dtype)
            out = layer(xx)
            experts_only = layer.experts(xx, *layer.router(xx))
            sh = layer.shared_expert(xx)
            k = layer.experts.args.moe_top_k
            ref = sh / (k + 1) + experts_only * (k / (k + 1)) if weighted else sh + experts_only
            torch.testing.assert_close(out.float(), ref.float(), **_tol(device))
            keys = set(layer.state_dict())
            assert {'shared_expert.up_proj.weight', 'shared_expert.down_proj.weight'} <= keys
            assert ('shared_expert.gate_proj.weight' in keys) == (typ == 'glu')


def test_state_dict_keys_and_shapes():
    E, h, f = 4, 128, 256
    for impl in ('sparse', 'grouped'):
        sd = mb.dMoE(_args('cpu', hs=h, ffn=f, ne=E, mlp_impl=impl, mlp_type='glu')).state_dict()
        assert {k: tuple(v.shape) for k, v in sd.items()} == {
            'router.layer.weight': (E, h), 'experts.bias': (h,), 'experts.mlp.w1': (E * f, h),
            'experts.mlp.w2': (E * f, h), 'experts.mlp.v1': (E * f, h)}
    sd = mb.MoE(_args('cpu', hs=h, ffn=f, ne=E)).state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        'router.layer.weight': (E, h), 'experts.bias': (h,), 'experts.mlp.w1': (E, h, f),
        'experts.mlp.w2': (E, f, h)}
    # Round trip through load_state_dict with reference-shaped tensors.
    src = mb.dMoE(_args('cpu', hs=h, ffn=f, ne=E))
    dst = mb.dMoE(_args('cpu', hs=h, ffn=f, ne=E))
    dst.load_state_dict({k: v.clone() for k, v in src.state_dict().items()})
    x = torch.randn(8, 1, h)
    torch.testing.assert_close(src(x)[0], dst(x)[0])


def test_same_seed_same_weights_any_impl():
    torch.manual_seed(7)
    a = mb.dMoE(_args('cpu', mlp_impl='sparse'))
    torch.manual_seed(7)
    b = mb.dMoE(_args('cpu', mlp_impl='grouped'))
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)


@pytest.mark.parametrize('device', DEVICES)
def test_losses(device):
    L = 3
    args = _args(device, ne=8, top_k=2, num_layers=L, moe_loss_weight=0.1, moe_zloss_weight=1e-3,
                 moe_lbl_in_fp32=True, moe_zloss_in_fp32=True)
    layers = [mb.dMoE(args) for _ in range(L)]
    x = torch.randn(16, 2, 128, device=device).to(layers[0].router.layer.weight.dtype)
    for layer in layers:
        layer.train()
        layer(x)
    lbl = moe_mod.batched_load_balancing_loss(args)
    zl = router_mod.batched_router_zloss(args)
    assert zl.shape == (L,)
    expected = 0.0
    for layer in layers:
        _, scores, e = dense_oracle(layer, x)
        tpe = torch.bincount(e.flatten(), minlength=8).float()
        expected = expected + (tpe * scores.mean(0)).sum()
    expected = expected * 8 * 0.1 / (L * 32 * 2)
    torch.testing.assert_close(lbl.float().cpu(), expected.cpu(), rtol=2e-2, atol=1e-3)
    logits = x.view(-1, 128).float() @ layers[0].router.layer.weight.float().t()
    torch.testing.assert_close(zl[0].float(), 1e-3 * torch.logsumexp(logits, 1).square().mean(), rtol=2e-2,
                               atol=1e-4)
    (lbl + zl.sum()).backward()
    assert layers[0].router.layer.weight.grad is not None
    with pytest.raises(ValueError):
        moe_mod.save_load_balancing_loss(moe_mod.get_load_balancing_loss()[0])
        moe_mod.batched_load_balancing_loss(args)
    moe_mod.clear_load_balancing_loss()
    router_mod.clear_router_zloss()
    assert moe_mod.get_load_balancing_loss() == []
    layers[0].eval()
    layers[0](x)
    assert moe_mod.get_load_balancing_loss() == []


@pytest.mark.parametrize('device', DEVICES)
def test_router_options(device):
    args = _args(device, ne=8, top_k=2, moe_normalize_expert_weights=1, moe_jitter_eps=0.1)
    layer = mb.dMoE(args)
    x = torch.randn(16, 2, 128, device=device).to(layer.router.layer.weight.dtype)
    layer.eval()
    scores, w, e = layer.router(x)
    torch.testing.assert_close(w.float().sum(-1), torch.ones(32, device=device), rtol=1e-2, atol=1e-2)
    assert scores.shape == (32, 8) and e.shape == (32, 2)
    layer.train()
    layer.router(x)  # jitter path
    uni = mb.dMoE(_args(device, ne=8, top_k=1, uniform_expert_assignment=True))
    _, _, e = uni.router(x.to(uni.router.layer.weight.dtype))
    assert torch.equal(e.flatten().cpu(), torch.arange(32) % 8)
    # top-1 ties resolve to the lowest expert id
    tie = mb.dMoE(_args(device, ne=4, top_k=1))
    with torch.no_grad():
        tie.router.layer.weight.zero_()
    _, _, e = tie.router(x.to(tie.router.layer.weight.dtype))
    assert int(e.max()) == 0


def test_arguments_defaults_and_from_megatron():
    a = mb.Arguments()
    assert (a.hidden_size, a.ffn_hidden_size, a.mlp_impl, a.mlp_type, a.fp16, a.bf16) == (1024, 4096, 'grouped',
                                                                                         'mlp', True, False)
    assert a.shared_expert_hidden_size == 4096 and a.moe_loss_weight == 0.1 and a.return_bias
    with pytest.raises(ValueError):
        mb.Arguments(mlp_impl='dense')

    class NS:
        hidden_size = 64
        moe_num_experts = 4
        unrelated = 1

    b = from_megatron(NS())
    assert b.hidden_size == 64 and b.moe_num_experts == 4


@pytest.mark.parametrize('device', DEVICES)
def test_custom_activation_callable(device):
    act = lambda t: F.relu(t) ** 2  # noqa: E731 - not known to the kernel: unfused route
    layer = mb.dMoE(_args(device, activation_fn=act, ne=4, top_k=2))
    x = torch.randn(8, 2, 128, device=device).to(layer.router.layer.weight.dtype).requires_grad_(True)
    out, _ = layer(x)
    ref, _, _ = dense_oracle(layer, x)
    torch.testing.assert_close(out.float(), ref, **_tol(device))
    out.float().sum().backward()
    assert layer.experts.mlp.w1.grad is not None
