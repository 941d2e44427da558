"""Fused cross-entropy and LayerNorm against the PyTorch ops in fp32."""

import pytest
import torch
import torch.nn.functional as F
from conftest import DEVICES

from megablocks_b200.ops import fused


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,vocab', [(64, 512), (257, 51200), (33, 1000), (8, 7)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_cross_entropy(device, rows, vocab, dtype):
    logits = (torch.randn(rows, vocab) * 3).to(dtype).to(device).requires_grad_(True)
    targets = torch.randint(0, vocab, (rows,), device=device)
    ref_in = logits.detach().float().cpu().requires_grad_(True)
    ref = F.cross_entropy(ref_in, targets.cpu())
    (ref * 1.7).backward()
    loss = fused.cross_entropy(logits, targets)
    torch.testing.assert_close(loss.float().cpu(), ref.detach(), rtol=1e-4, atol=1e-4)
    (loss * 1.7).backward()
    tol = dict(rtol=2e-2, atol=1e-4) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(logits.grad.float().cpu(), ref_in.grad, **tol)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,cols', [(1000, 768), (77, 1024), (4096, 128), (5, 4096)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_layer_norm(device, rows, cols, dtype):
    ln = fused.LayerNorm(cols).to(device=device, dtype=dtype)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(cols) * 0.5 + 1)
        ln.bias.copy_(torch.randn(cols) * 0.5)
    x = (torch.randn(rows, cols) * 2 + 0.3).to(dtype).to(device).requires_grad_(True)
    probe = torch.randn(rows, cols).to(dtype).to(device)
    y = ln(x)
    (y.float() * probe.float()).sum().backward()
    xr = x.detach().float().cpu().requires_grad_(True)
    wr = ln.weight.detach().float().cpu().requires_grad_(True)
    br = ln.bias.detach().float().cpu().requires_grad_(True)
    yr = F.layer_norm(xr, (cols,), wr, br, ln.eps)
    (yr * probe.float().cpu()).sum().backward()
    tol = dict(rtol=2e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(y.detach().float().cpu(), yr.detach(), **tol)
    torch.testing.assert_close(x.grad.float().cpu(), xr.grad, **tol)
    wtol = dict(rtol=3e-2, atol=3e-2 * float(wr.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(ln.weight.grad.float().cpu(), wr.grad, **wtol)
    torch.testing.assert_close(ln.bias.grad.float().cpu(), br.grad, **wtol)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,cols', [(1000, 768), (77, 1024), (64, 4096)])   # last: too wide to fuse, falls back
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_add_layer_norm(device, rows, cols, dtype):
    """``(a + b, LN(a + b))`` with both results used downstream, against the unfused fp32 chain."""
    ln = fused.LayerNorm(cols).to(device=device, dtype=dtype)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(cols) * 0.5 + 1)
        ln.bias.copy_(torch.randn(cols) * 0.5)
    a = torch.randn(rows, cols).to(dtype).to(device).requires_grad_(True)
    b = (torch.randn(rows, cols) * 0.5).to(dtype).to(device).requires_grad_(True)
    p1 = torch.randn(rows, cols).to(dtype).to(device)
    p2 = torch.randn(rows, cols).to(dtype).to(device)
    s, y = ln.add_forward(a, b)
    ((y.float() * p1.float()).sum() + (s.float() * p2.float()).sum()).backward()
    ar = a.detach().float().cpu().requires_grad_(True)
    br = b.detach().float().cpu().requires_grad_(True)
    sr = (ar + br).to(dtype).float() if dtype == torch.bfloat16 else ar + br
    # Straight-through for the rounding of the sum, as autograd sees the 16-bit add.
    sr = (ar + br) + (sr - (ar + br)).detach()
    yr = F.layer_norm(sr, (cols,), ln.weight.detach().float().cpu(), ln.bias.detach().float().cpu(), ln.eps)
    ((yr * p1.float().cpu()).sum() + (sr * p2.float().cpu()).sum()).backward()
    tol = dict(rtol=2e-2, atol=4e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s.detach().float().cpu(), sr.detach(), **tol)
    torch.testing.assert_close(y.detach().float().cpu(), yr.detach(), **tol)
    torch.testing.assert_close(a.grad.float().cpu(), ar.grad, **tol)
    torch.testing.assert_close(b.grad.float().cpu(), br.grad, **tol)
    # Only the normalised output used: the residual gradient is absent.
    a.grad = b.grad = None
    s2, y2 = ln.add_forward(a, b)
    (y2.float() * p1.float()).sum().backward()
    assert a.grad is not None and torch.equal(a.grad, b.grad)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,cin,cout', [(1000, 64, 768), (4099, 128, 2304), (7, 32, 8)])
def test_linear_bias_gradient(device, rows, cin, cout):
    """``fused.Linear`` against ``nn.Linear`` in fp32: outputs and all three gradients."""
    dtype = torch.bfloat16 if device == 'cuda' else torch.float32
    lin = fused.Linear(cin, cout).to(device=device, dtype=dtype)
    x = torch.randn(rows, cin).to(dtype).to(device).requires_grad_(True)
    probe = torch.randn(rows, cout).to(dtype).to(device)
    y = lin(x)
    (y.float() * probe.float()).sum().backward()
    xr = x.detach().float().cpu().requires_grad_(True)
    wr = lin.weight.detach().float().cpu().requires_grad_(True)
    br = lin.bias.detach().float().cpu().requires_grad_(True)
    (F.linear(xr, wr, br) * probe.float().cpu()).sum().backward()
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(y.detach().float().cpu(), F.linear(xr, wr, br).detach(), **tol)
    torch.testing.assert_close(x.grad.float().cpu(), xr.grad, **tol)
    scale = dict(rtol=2e-2, atol=2e-2 * float(br.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(lin.bias.grad.float().cpu(), br.grad, **scale)
    wscale = dict(rtol=2e-2, atol=2e-2 * float(wr.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(lin.weight.grad.float().cpu(), wr.grad, **wscale)
