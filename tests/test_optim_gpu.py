"""The CUDA optimizer kernels against ``torch.optim.Adam`` and plain fp32 formulas.

``adam_kernel`` (multi-tensor Adam with fp32 master weights and a 16-bit shadow), ``sqnorm_kernel``
(weighted squared gradient norm) and ``clip_coeff`` are compared with an fp32 reference run on
the same gradients: ``torch.optim.Adam`` on fp32 copies of the parameters, with the gradients
multiplied by the clip coefficient the reference formula gives.
"""

import pytest
import torch

from megablocks_b200.optim import FusedAdam, clip_coefficient


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('weight_decay', [0.0, 0.1])
def test_fused_adam_kernel_matches_torch_adam(dtype, weight_decay):
    dev = torch.device('cuda', 0)
    torch.manual_seed(0)
    shapes = [(257, 129), (65536 + 8,), (3,), (1024, 768), (7, 5, 3)]      # spans several 65536-element chunks, odd tails
    params = [torch.randn(*s, device=dev).mul(0.1).to(dtype).requires_grad_(True) for s in shapes]
    masters = [p.detach().float().clone().requires_grad_(True) for p in params]
    opt = FusedAdam(params, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=weight_decay,
                    norm_weights=[1.0, 0.5, 1.0, 0.25, 1.0])
    # FusedAdam applies decoupled decay w -= lr * wd * w (AdamW).
    ref = torch.optim.AdamW(masters, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=weight_decay)
    sq = torch.zeros(1, dtype=torch.float32, device=dev)
    for step in range(5):
        grads = [torch.randn_like(p).mul(0.5 + step) for p in params]
        for p, g in zip(params, grads):
            p.grad = g
        # squared norm with per-tensor weights, fp32 oracle from the (rounded) gradients
        sq.zero_()
        opt.add_sqnorm(sq)
        want_sq = sum(w * g.float().square().sum() for w, g in zip(opt.norm_weights, grads))
        torch.testing.assert_close(sq[0], want_sq, rtol=1e-4, atol=1e-6)
        coeff = clip_coefficient(sq, max_norm=1.0)
        norm = float(want_sq.sqrt())
        torch.testing.assert_close(coeff.cpu(), torch.tensor([min(1.0, 1.0 / (norm + 1e-6)), norm]), rtol=1e-4,
                                   atol=1e-6)
        opt.step(coeff[0:1])
        for m, g in zip(masters, grads):
            m.grad = g.float() * float(coeff[0])
        ref.step()
    torch.cuda.synchronize()
    for i, (p, m) in enumerate(zip(params, masters)):
        n = p.numel()
        off = opt.offsets[i]
        # fp32 master weights follow torch's Adam closely; the 16-bit shadow is their rounding.
        torch.testing.assert_close(opt.master[off:off + n].view_as(m), m.detach(), rtol=1e-4, atol=1e-5)
        assert torch.equal(p.detach(), opt.master[off:off + n].view_as(p).to(dtype))


@pytest.mark.gpu
def test_clip_coefficient_zero_on_overflow():
    dev = torch.device('cuda', 0)
    coeff = clip_coefficient(torch.tensor([float('inf')], device=dev), 1.0)
    assert float(coeff[0]) == 0.0
    coeff = clip_coefficient(torch.tensor([4.0], device=dev), 1.0, extra_scale=0.5)
    torch.testing.assert_close(coeff.cpu(), torch.tensor([0.25, 2.0]), rtol=1e-5, atol=1e-6)
