"""Checkpoint and numerics interoperability with the installed reference library (GPU).

A ``dMoE`` of the reference (``baseline/_ref``, imported through its public API) and a
``megablocks_b200.dMoE`` are built from the same ``Arguments`` values; the reference layer's
``state_dict()`` is loaded into this library's layer (and back), both get the same input, and
outputs, input gradients and every parameter gradient must agree - the weight-copy idiom of the
reference's own layer test (tests/layers/dmoe_test.py:91-99 of the reference).  Skipped when
the reference is not installed next to the repository.
"""

import os
import sys
from functools import partial

import pytest
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference():
    sys.path.insert(0, os.path.join(ROOT, 'baseline'))
    try:
        import ref_arm
        return ref_arm.import_reference()
    except Exception as exc:   # not installed, or its extension does not load on this machine
        pytest.skip(f'reference library unavailable: {type(exc).__name__}: {exc}')


@pytest.mark.gpu
@pytest.mark.parametrize('mlp_type,top_k', [('mlp', 1), ('mlp', 2), ('glu', 2)])
def test_state_dict_round_trip_and_equal_results(mlp_type, top_k):
    RefArguments, ref_dmoe, ref_moe = _reference()
    import megablocks_b200 as mb
    dev = torch.device('cuda', 0)
    common = dict(hidden_size=256, ffn_hidden_size=512, moe_num_experts=8, moe_top_k=top_k, bias=True,
                  return_bias=False, activation_fn=partial(F.gelu, approximate='tanh'), moe_loss_weight=0.0,
                  mlp_type=mlp_type, mlp_impl='grouped', fp16=False, bf16=True, device=dev,
                  init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.1))
    torch.manual_seed(0)
    theirs = ref_dmoe.dMoE(RefArguments(**common))
    torch.manual_seed(1)
    ours = mb.dMoE(mb.Arguments(**common))

    state = theirs.state_dict()
    assert set(state) == set(ours.state_dict()), 'parameter names differ from the reference'
    ours.load_state_dict(state)                                   # reference checkpoint -> this library
    theirs.load_state_dict(ours.state_dict())                     # and back
    for name, value in theirs.state_dict().items():
        assert torch.equal(value, state[name]), name

    torch.manual_seed(2)
    x = torch.randn(64, 4, 256, device=dev, dtype=torch.bfloat16)
    probe = torch.randn_like(x)
    results = []
    for layer in (theirs, ours):
        xi = x.clone().requires_grad_(True)
        out = layer(xi)
        (out.float() * probe.float()).sum().backward()
        results.append((out.detach().float(), xi.grad.float(), {n: p.grad.float() for n, p in layer.named_parameters()}))
    ref_moe.clear_load_balancing_loss()
    (out_t, dx_t, g_t), (out_o, dx_o, g_o) = results

    def close(a, b, what):
        torch.testing.assert_close(a, b, rtol=3e-2, atol=2e-2 * float(b.abs().max()) + 1e-3, msg=lambda m: f'{what}: {m}')

    close(out_o, out_t, 'output')
    close(dx_o, dx_t, 'input gradient')
    for name in g_t:
        close(g_o[name], g_t[name], name)
