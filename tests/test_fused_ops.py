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
@pytest.mark.parametrize('rows,cols', [(1000, 768), (333, 1024), (64, 4096)])   # last: too wide to fuse, falls back
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_add_layer_norm_with_the_bias_of_the_added_tensor(device, rows, cols, dtype):
    """``s = a + b + v`` (``v`` one value per column), ``LN(s)``, and the gradient of ``v`` (a column sum
    of the gradient of ``s``), against the unfused fp32 chain."""
    ln = fused.LayerNorm(cols).to(device=device, dtype=dtype)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(cols) * 0.5 + 1)
        ln.bias.copy_(torch.randn(cols) * 0.5)
    a = torch.randn(rows, cols).to(dtype).to(device).requires_grad_(True)
    b = (torch.randn(rows, cols) * 0.5).to(dtype).to(device).requires_grad_(True)
    v = (torch.randn(cols) * 0.5).to(dtype).to(device).requires_grad_(True)
    p1 = (torch.randn(rows, cols) / rows**0.5).to(dtype).to(device)
    p2 = (torch.randn(rows, cols) / rows**0.5).to(dtype).to(device)
    s, y = ln.add_forward(a, b, v)
    ((y.float() * p1.float()).sum() + (s.float() * p2.float()).sum()).backward()
    ar, br, vr = (t.detach().float().cpu().requires_grad_(True) for t in (a, b, v))
    exact = ar + br + vr
    sr = exact + ((exact.to(dtype).float() if dtype == torch.bfloat16 else exact) - exact).detach()
    yr = F.layer_norm(sr, (cols,), ln.weight.detach().float().cpu(), ln.bias.detach().float().cpu(), ln.eps)
    ((yr * p1.float().cpu()).sum() + (sr * p2.float().cpu()).sum()).backward()
    tol = dict(rtol=2e-2, atol=4e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s.detach().float().cpu(), sr.detach(), **tol)
    torch.testing.assert_close(y.detach().float().cpu(), yr.detach(), **tol)
    gtol = dict(rtol=2e-2, atol=4e-2 / rows**0.5) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(a.grad.float().cpu(), ar.grad, **gtol)
    torch.testing.assert_close(b.grad.float().cpu(), br.grad, **gtol)
    vtol = dict(rtol=3e-2, atol=3e-2 * float(vr.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(v.grad.float().cpu(), vr.grad, **vtol)


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


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,cols', [(1000, 768), (77, 1024), (300, 4096), (64, 128)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_rms_norm_and_fused_add(device, rows, cols, dtype):
    """RMS norm (and the residual-add form) forward and backward against the fp32 formula."""
    norm = fused.RMSNorm(cols, eps=1e-5).to(device=device, dtype=dtype)
    with torch.no_grad():
        norm.weight.copy_(torch.randn(cols) * 0.5 + 1)
    a = (torch.randn(rows, cols) * 2 + 0.3).to(dtype).to(device).requires_grad_(True)
    b = torch.randn(rows, cols).to(dtype).to(device).requires_grad_(True)
    p1 = torch.randn(rows, cols).to(dtype).to(device)
    p2 = torch.randn(rows, cols).to(dtype).to(device)

    def ref_norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w

    tol = dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    y = norm(a)
    (y.float() * p1.float()).sum().backward()
    ar = a.detach().float().cpu().requires_grad_(True)
    wr = norm.weight.detach().float().cpu().requires_grad_(True)
    (ref_norm(ar, wr) * p1.float().cpu()).sum().backward()
    torch.testing.assert_close(y.detach().float().cpu(), ref_norm(ar, wr).detach(), **tol)
    torch.testing.assert_close(a.grad.float().cpu(), ar.grad, **tol)
    wtol = dict(rtol=3e-2, atol=3e-2 * float(wr.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(norm.weight.grad.float().cpu(), wr.grad, **wtol)

    # (a + b, norm(a + b)) with gradients arriving on both outputs.
    a.grad = None
    norm.weight.grad = None
    s, y = norm.add_forward(a, b)
    ((y.float() * p1.float()).sum() + (s.float() * p2.float()).sum()).backward()
    ar = a.detach().float().cpu().requires_grad_(True)
    br = b.detach().float().cpu().requires_grad_(True)
    sr = (ar + br).to(dtype).float() if dtype == torch.bfloat16 else ar + br
    sr_live = ar + br
    ((ref_norm(sr_live, wr.detach()) * p1.float().cpu()).sum() + (sr_live * p2.float().cpu()).sum()).backward()
    torch.testing.assert_close(s.detach().float().cpu(), sr.detach(), **tol)
    torch.testing.assert_close(a.grad.float().cpu(), ar.grad, **tol)
    torch.testing.assert_close(b.grad.float().cpu(), br.grad, **tol)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('batch,seq,heads,dim', [(2, 64, 4, 32), (1, 300, 8, 128), (3, 17, 2, 64)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_rope(device, batch, seq, heads, dim, dtype):
    """Rotary embedding of a strided [batch, seq, heads, dim] view (a slice of a fused projection)."""
    qkv = torch.randn(batch, seq, 3 * heads * dim).to(dtype).to(device).requires_grad_(True)
    inv = 1.0 / (10000.0**(torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    cos, sin = ang.cos().to(device), ang.sin().to(device)
    k = qkv[..., heads * dim:2 * heads * dim].view(batch, seq, heads, dim)      # non-contiguous view
    out = fused.rope(k, cos, sin)
    probe = torch.randn(batch, seq, heads, dim).to(dtype).to(device)
    (out.float() * probe.float()).sum().backward()

    ref_in = qkv.detach().float().cpu().requires_grad_(True)
    kr = ref_in[..., heads * dim:2 * heads * dim].view(batch, seq, heads, dim)
    half = dim // 2
    c, s = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    ref = torch.cat([kr[..., :half] * c - kr[..., half:] * s, kr[..., half:] * c + kr[..., :half] * s], dim=-1)
    (ref * probe.float().cpu()).sum().backward()
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.detach().float().cpu(), ref.detach(), **tol)
    torch.testing.assert_close(qkv.grad.float().cpu(), ref_in.grad, **tol)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('layers,tokens,experts,top_k', [(1, 64, 8, 1), (12, 4096, 64, 1), (3, 1000, 48, 2),
                                                         (2, 300, 512, 4)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_batched_load_balancing_loss(device, layers, tokens, experts, top_k, dtype):
    """All layers' auxiliary loss (one reduction kernel on CUDA) against the concatenated fp32 formula."""
    import megablocks_b200 as mb
    from megablocks_b200.layers import moe
    args = mb.Arguments(hidden_size=64, ffn_hidden_size=64, num_layers=layers, moe_num_experts=experts, moe_top_k=top_k,
                        moe_loss_weight=0.1, moe_lbl_in_fp32=True, device=torch.device(device))
    scores = [torch.softmax(torch.randn(tokens, experts), -1).to(dtype).to(device).requires_grad_(True)
              for _ in range(layers)]
    counts = [torch.bincount(torch.randint(0, experts, (tokens * top_k,)), minlength=experts).int().to(device)
              for _ in range(layers)]
    moe.clear_load_balancing_loss()
    for c, s in zip(counts, scores):
        moe.save_load_balancing_loss((c, s))
    loss = moe.batched_load_balancing_loss(args)
    (loss * 3.0).backward()
    moe.clear_load_balancing_loss()

    ref_scores = [s.detach().float().cpu().requires_grad_(True) for s in scores]
    cat_scores = torch.cat(ref_scores, dim=1).mean(dim=0)
    cat_counts = torch.cat([c.cpu() for c in counts]).float()
    ref = experts * 0.1 / (layers * tokens * top_k) * torch.dot(cat_counts, cat_scores)
    (ref * 3.0).backward()
    torch.testing.assert_close(loss.detach().float().cpu(), ref.detach(), rtol=1e-3, atol=1e-6)
    for s, r in zip(scores, ref_scores):
        torch.testing.assert_close(s.grad.float().cpu(), r.grad, rtol=1e-2, atol=1e-9)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('rows,hidden,vocab', [(64, 32, 1000), (300, 64, 5003), (1024, 128, 51200)])
def test_linear_cross_entropy_matches_the_unfused_head_and_loss(device, rows, hidden, vocab):
    """LM head + mean cross entropy with loss and logit gradient in one pass, against F.linear +
    F.cross_entropy in fp32: loss, both gradients, an upstream gradient other than one, ignored rows."""
    if device == 'cpu' and vocab > 10000:
        pytest.skip('large vocabulary on the GPU only')
    dtype = torch.bfloat16 if device == 'cuda' else torch.float32
    h = (torch.randn(rows, hidden) * 0.5).to(dtype).to(device).requires_grad_(True)
    w = (torch.randn(vocab, hidden) * 0.2).to(dtype).to(device).requires_grad_(True)
    t = torch.randint(0, vocab, (rows,)).to(device)
    loss = fused.linear_cross_entropy(h, w, t)
    (loss * 3.0).backward()
    hr, wr = h.detach().float().cpu().requires_grad_(True), w.detach().float().cpu().requires_grad_(True)
    logits = F.linear(hr, wr)
    if dtype == torch.bfloat16:      # the fused path sees the logits rounded to bf16
        logits = logits + (logits.to(dtype).float() - logits).detach()
    ref = F.cross_entropy(logits, t.cpu())
    (ref * 3.0).backward()
    tol = dict(rtol=2e-2, atol=2e-3) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(loss.detach().float().cpu(), ref.detach(), rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(h.grad.float().cpu(), hr.grad, **tol)
    wtol = dict(rtol=3e-2, atol=3e-2 * float(wr.grad.abs().max())) if dtype == torch.bfloat16 else tol
    torch.testing.assert_close(w.grad.float().cpu(), wr.grad, **wtol)
