"""Grouped GEMM (all layouts and fused epilogues) against per-group fp32 matmuls."""

import pytest
import torch
import torch.nn.functional as F
from conftest import DEVICES

from megablocks_b200.ops import gg as G


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-4, atol=1e-4)


def _close(out, ref, dtype):
    """Compare against an fp32 reference; a 16-bit result carries one rounding of its own magnitude."""
    out, ref = out.detach().cpu().float(), ref.detach().cpu().float()
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    else:
        torch.testing.assert_close(out, ref, rtol=2e-2, atol=1e-2 * float(ref.abs().max()) + 1e-3)


def _dtype_for(device):
    return torch.bfloat16 if device == 'cuda' else torch.float32


def _sizes(z, m, device, zipf=False):
    if zipf:
        p = 1.0 / torch.arange(1, z + 1).float()**1.1
        idx = torch.multinomial(p / p.sum(), m, replacement=True)
    else:
        idx = torch.randint(0, z, (m,))
    counts = torch.bincount(idx, minlength=z)
    return counts, torch.cumsum(counts, 0).int().to(device)


def _ref_gmm(a, b, counts, trans_b):
    out, start = [], 0
    for e, c in enumerate(counts.tolist()):
        w = b[e].float()
        out.append(a[start:start + c].float() @ (w.t() if trans_b else w))
        start += c
    return torch.cat(out)


SHAPES = [(1, 128, 128, 128), (8, 1024, 256, 512), (4, 777, 192, 320), (16, 4096, 768, 3072), (64, 8192, 768, 3072),
          (3, 100, 64, 64), (300, 6000, 64, 128)]   # last: more groups than the kernel's small tables hold


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('z,m,k,n', SHAPES)
@pytest.mark.parametrize('trans_b', [False, True])
def test_gmm_forward_backward(device, z, m, k, n, trans_b):
    if device == 'cpu' and m * k * n > 2**31:
        pytest.skip('large case is GPU-only')
    dtype = _dtype_for(device)
    counts, bins = _sizes(z, m, device, zipf=(z == 16))
    a = (torch.randn(m, k) * 0.5).to(dtype).to(device).requires_grad_(True)
    b = (torch.randn(z, n, k) if trans_b else torch.randn(z, k, n)).mul(0.1).to(dtype).to(device).requires_grad_(True)
    out = G.gmm_bins(a, b, bins, trans_b)
    a2 = a.detach().cpu().float().requires_grad_(True)
    b2 = b.detach().cpu().float().requires_grad_(True)
    ref = _ref_gmm(a2, b2, counts, trans_b)
    _close(out, ref, dtype)
    probe = torch.randn(m, n).to(dtype).float()
    (out.float() * probe.to(device)).sum().backward()
    (ref * probe).sum().backward()
    _close(a.grad, a2.grad, dtype)
    _close(b.grad, b2.grad, dtype)


@pytest.mark.parametrize('device', DEVICES)
def test_gmm_batch_sizes_signature(device):
    dtype = _dtype_for(device)
    counts = torch.tensor([3, 0, 5, 120])
    a = torch.randn(128, 64).to(dtype).to(device)
    b = torch.randn(4, 64, 128).mul(0.1).to(dtype).to(device)
    out = G.gmm(a, b, counts)
    torch.testing.assert_close(out.cpu().float(), _ref_gmm(a.cpu(), b.cpu(), counts, False), **_tol(dtype))
    raw = G.backend.gmm(a, b, counts)
    assert torch.equal(raw, out)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('act', [G.ACT_GELU_TANH, G.ACT_SILU, G.ACT_RELU, G.ACT_GELU_ERF, G.ACT_IDENTITY])
def test_epilogues(device, act):
    dtype = _dtype_for(device)
    z, m, k, n = 4, 600, 128, 256
    counts, bins = _sizes(z, m, device)
    a = torch.randn(m, k).mul(0.5).to(dtype).to(device)
    w = torch.randn(z, n, k).mul(0.2).to(dtype).to(device)
    acc = _ref_gmm(a.cpu(), w.cpu(), counts, True)
    tol = _tol(dtype)

    c, h, _ = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_ACT, act=act)
    torch.testing.assert_close(c.cpu().float(), acc, **tol)
    torch.testing.assert_close(h.cpu().float(), G.act_forward(c.cpu().float(), act), **tol)

    z1 = torch.randn(m, n).to(dtype).to(device)
    z2 = torch.randn(m, n).to(dtype).to(device)
    z1f, z2f = z1.cpu().float(), z2.cpu().float()
    zz = z1f.clone().requires_grad_(True)
    G.act_forward(zz, act).sum().backward()
    dact = zz.grad

    c, h, _ = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_DACT, act=act, aux1=z1)
    torch.testing.assert_close(c.cpu().float(), acc * dact, **tol)
    torch.testing.assert_close(h.cpu().float(), G.act_forward(z1f, act), **tol)

    c, h, _ = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_GLU, act=act, aux1=z1)
    torch.testing.assert_close(c.cpu().float(), acc, **tol)
    torch.testing.assert_close(h.cpu().float(), G.act_forward(z1f, act) * c.cpu().float(), **tol)

    c, d2, h = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_DGLU, act=act, aux1=z1, aux2=z2)
    torch.testing.assert_close(c.cpu().float(), acc * z2f * dact, **tol)
    torch.testing.assert_close(d2.cpu().float(), acc * G.act_forward(z1f, act), **tol)
    torch.testing.assert_close(h.cpu().float(), G.act_forward(z1f, act) * z2f, **tol)

    c, _, _ = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_ADD, aux1=z1)
    torch.testing.assert_close(c.cpu().float(), acc + z1f, **tol)


@pytest.mark.parametrize('device', DEVICES)
def test_rows_past_last_bin_are_zero(device):
    dtype = _dtype_for(device)
    a = torch.randn(512, 128).to(dtype).to(device)
    w = torch.randn(2, 128, 128).mul(0.1).to(dtype).to(device)
    bins = torch.tensor([128, 256], dtype=torch.int32, device=device)
    out, _, _ = G.grouped_gemm(a, w, bins)
    assert not out[256:].any()
    ref = _ref_gmm(a.cpu()[:256], w.cpu(), torch.tensor([128, 128]), False)
    torch.testing.assert_close(out[:256].cpu().float(), ref, **_tol(dtype))


def test_activation_id():
    from functools import partial
    assert G.activation_id(partial(F.gelu, approximate='tanh')) == G.ACT_GELU_TANH
    assert G.activation_id(F.gelu) == G.ACT_GELU_ERF
    assert G.activation_id(F.silu) == G.ACT_SILU
    assert G.activation_id(torch.nn.ReLU()) == G.ACT_RELU
    assert G.activation_id(lambda t: t * 2) is None
    for act in (G.ACT_GELU_TANH, G.ACT_SILU, G.ACT_GELU_ERF):
        zz = torch.randn(1000, dtype=torch.float64, requires_grad=True)
        G.act_forward(zz, act).sum().backward()
        torch.testing.assert_close(G.act_derivative(zz.detach(), act), zz.grad, rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
def test_cta_pair_kernel_matches_reference():
    """The cta_group::2 kernel (256-row tiles on CTA pairs), forced on through its environment switch."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from megablocks_b200.ops import gg as G
from megablocks_b200.utils import status
torch.manual_seed(0)
dev = 'cuda'
for z, m, k, n in [(1, 128, 128, 256), (3, 1000, 192, 320), (5, 3000, 256, 512), (8, 8192, 768, 3072)]:
    counts = torch.bincount(torch.randint(0, z, (m,)), minlength=z)
    bins = torch.cumsum(counts, 0).int().to(dev)
    a = (torch.randn(m, k) * 0.5).bfloat16().to(dev)
    for trans_b in (True, False):
        b = (torch.randn(z, n, k) if trans_b else torch.randn(z, k, n)).mul(0.1).bfloat16().to(dev)
        aux = torch.randn(m, n).bfloat16().to(dev)
        out, h, _ = G.grouped_gemm(a, b, bins, trans_b=trans_b, epilogue=G.EPI_DACT, act=G.ACT_GELU_TANH, aux1=aux)
        ref, start = [], 0
        for e, c in enumerate(counts.tolist()):
            w = b[e].float()
            ref.append(a[start:start + c].float() @ (w.t() if trans_b else w))
            start += c
        ref = torch.cat(ref).cpu()
        zz = aux.float().cpu().requires_grad_(True)
        G.act_forward(zz, G.ACT_GELU_TANH).sum().backward()
        want = ref * zz.grad
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=1e-2 * float(want.abs().max()) + 1e-3)
        torch.testing.assert_close(h.float().cpu(), G.act_forward(aux.float().cpu(), G.ACT_GELU_TANH), rtol=2e-2, atol=2e-2)
status.check()
print('PAIR-OK')
'''
    env = dict(os.environ, MB200_GEMM_PAIR='1')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env['PYTHONPATH'] = root + os.pathsep + env.get('PYTHONPATH', '')
    res = subprocess.run([sys.executable, '-c', code], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and 'PAIR-OK' in res.stdout, res.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize('z,rows,m,n', [(1, 64, 256, 256), (3, 1000, 320, 256), (5, 3000, 768, 512),
                                        (8, 8192, 3072, 768), (6, 200, 128, 384), (64, 4096, 256, 1024)])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_cta_pair_weight_gradient(z, rows, m, n, dtype):
    """TN (ragged-K) layout on CTA pairs against per-group fp32 products; some groups are empty."""
    from megablocks_b200.utils import status
    torch.manual_seed(z * 1000 + rows)
    idx = torch.randint(0, z, (rows,))
    if z > 2:
        idx[idx == 1] = 0                       # an empty group in the middle
    if z > 3:
        idx[idx == z - 1] = z - 2               # and an empty last group
    counts = torch.bincount(idx, minlength=z)
    bins = torch.cumsum(counts, 0).int().cuda()
    # Rows past the last group exist in the buffers and hold NaN: they must not contribute.
    a = torch.full((rows + 70, m), float('nan'), dtype=dtype, device='cuda')
    b = torch.full((rows + 70, n), float('nan'), dtype=dtype, device='cuda')
    a[:rows] = (torch.randn(rows, m) * 0.5).to(dtype)
    b[:rows] = (torch.randn(rows, n) * 0.5).to(dtype)
    out, _, _ = G.grouped_gemm(a, b, bins, trans_a=True, num_groups=z, alpha=0.5, pair=1)
    single, _, _ = G.grouped_gemm(a, b, bins, trans_a=True, num_groups=z, alpha=0.5, pair=0)
    ref, start = [], 0
    for c in counts.tolist():
        ref.append(a[start:start + c].float().cpu().t() @ b[start:start + c].float().cpu() * 0.5)
        start += c
    ref = torch.stack(ref)
    status.check()
    _close(out, ref, dtype)
    _close(single, ref, dtype)


@pytest.mark.gpu
def test_cta_pair_short_groups():
    """Pair tiles whose second half holds no rows of the group (its A tile is not loaded)."""
    from megablocks_b200.utils import status
    torch.manual_seed(5)
    counts = torch.tensor([100, 0, 300, 129, 128, 1, 512, 257])
    z, m, k, n = counts.numel(), int(counts.sum()), 256, 512
    bins = torch.cumsum(counts, 0).int().cuda()
    a = (torch.randn(m, k) * 0.5).bfloat16().cuda()
    for trans_b in (True, False):
        b = (torch.randn(z, n, k) if trans_b else torch.randn(z, k, n)).mul(0.1).bfloat16().cuda()
        out, _, _ = G.grouped_gemm(a, b, bins, trans_b=trans_b, pair=1)
        status.check()
        _close(out, _ref_gmm(a.cpu(), b.cpu(), counts, trans_b), torch.bfloat16)


@pytest.mark.gpu
def test_bins_outside_the_operand_are_clamped():
    """Group ends beyond the row count (or decreasing) never make the kernel touch rows that do not exist."""
    from megablocks_b200.utils import status
    a = (torch.randn(256, 128) * 0.5).bfloat16().cuda()
    w = (torch.randn(3, 128, 128) * 0.1).bfloat16().cuda()
    guard = torch.zeros(4096, 128, dtype=torch.bfloat16, device='cuda')
    c = guard[:256]
    bins = torch.tensor([128, 64, 100000], dtype=torch.int32, device='cuda')     # treated as [128, 128, 256]
    G.grouped_gemm(a, w, bins, trans_b=True, c=c)
    status.check()
    assert not guard[256:].any()
    ref = torch.cat([a[:128].float() @ w[0].float().t(), a[128:].float() @ w[2].float().t()])
    _close(c, ref, torch.bfloat16)


@pytest.mark.parametrize('device', DEVICES)
def test_alpha_scales_the_accumulators(device):
    """``alpha`` multiplies the product before the epilogue: NT output and TN (ragged-K) weight gradient."""
    dtype = _dtype_for(device)
    z, m, k, n = 4, 700, 128, 256
    counts, bins = _sizes(z, m, device)
    a = torch.randn(m, k).mul(0.5).to(dtype).to(device)
    w = torch.randn(z, n, k).mul(0.2).to(dtype).to(device)
    plain, _, _ = G.grouped_gemm(a, w, bins, trans_b=True)
    scaled, _, _ = G.grouped_gemm(a, w, bins, trans_b=True, alpha=0.25)
    _close(scaled, _ref_gmm(a.cpu(), w.cpu(), counts, True) * 0.25, dtype)
    _close(scaled, plain.float() * 0.25, dtype)
    g = torch.randn(m, n).mul(0.5).to(dtype).to(device)
    dw, _, _ = G.grouped_gemm(g, a, bins, trans_a=True, num_groups=z, alpha=0.125)
    ref, start = [], 0
    for c in counts.tolist():
        ref.append(g[start:start + c].float().cpu().t() @ a[start:start + c].float().cpu())
        start += c
    _close(dw, torch.stack(ref) * 0.125, dtype)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('z,m,k,n', [(4, 600, 128, 256), (3, 1000, 192, 384), (8, 4096, 256, 1024), (2, 130, 64, 200)])
@pytest.mark.parametrize('act', [G.ACT_SILU, G.ACT_GELU_TANH])
def test_glu_forward_in_one_launch(device, z, m, k, n, act):
    """Two weight operands per tile: (x v^T, act(x w^T) * (x v^T), x w^T) against per-group fp32 products."""
    dtype = _dtype_for(device)
    counts, bins = _sizes(z, m, device)
    a = torch.randn(m, k).mul(0.5).to(dtype).to(device)
    w = torch.randn(z, n, k).mul(0.2).to(dtype).to(device)
    v = torch.randn(z, n, k).mul(0.2).to(dtype).to(device)
    z2, h, z1 = G.grouped_gemm(a, w, bins, trans_b=True, epilogue=G.EPI_GLU_DUAL, act=act, b2=v)
    r1 = _ref_gmm(a.cpu(), w.cpu(), counts, True)
    r2 = _ref_gmm(a.cpu(), v.cpu(), counts, True)
    _close(z1, r1, dtype)
    _close(z2, r2, dtype)
    want_h = G.act_forward(z1.detach().cpu().float(), act) * z2.detach().cpu().float()   # from the rounded outputs
    _close(h, want_h, dtype)
    if device == 'cuda':
        # Same numbers as the two-launch form.
        s1, _, _ = G.grouped_gemm(a, w, bins, trans_b=True)
        s2, sh, _ = G.grouped_gemm(a, v, bins, trans_b=True, epilogue=G.EPI_GLU, act=act, aux1=s1)
        assert torch.equal(s1, z1) and torch.equal(s2, z2) and torch.equal(sh, h)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('z,m,k,n', [(4, 600, 256, 128), (3, 1000, 320, 192), (8, 4096, 1024, 256), (2, 130, 72, 64)])
def test_two_operand_pairs_in_one_contraction(device, z, m, k, n):
    """c = a b + a2 b2 (the GLU input gradient) against per-group fp32 products."""
    dtype = _dtype_for(device)
    counts, bins = _sizes(z, m, device)
    a = torch.randn(m, k).mul(0.5).to(dtype).to(device)
    a2 = torch.randn(m, k).mul(0.5).to(dtype).to(device)
    b = torch.randn(z, k, n).mul(0.1).to(dtype).to(device)
    b2 = torch.randn(z, k, n).mul(0.1).to(dtype).to(device)
    out, _, _ = G.grouped_gemm(a, b, bins, a2=a2, b2=b2)
    ref = _ref_gmm(a.cpu(), b.cpu(), counts, False) + _ref_gmm(a2.cpu(), b2.cpu(), counts, False)
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize('z,rows,m,n', [(4, 700, 128, 256), (8, 4096, 3072, 768), (5, 900, 200, 72), (64, 8192, 768, 3072)])
def test_weight_gradient_launch_reports_its_squared_norm(z, rows, m, n):
    """With a sink installed, a TN launch adds the sum of squares of what it stores to a slot of its own
    (odd shapes: clipped rows and columns must not contribute; empty groups store zeros)."""
    dtype = torch.bfloat16
    idx = torch.randint(0, z, (rows,))
    if z > 2:
        idx[idx == 1] = 0
    counts = torch.bincount(idx, minlength=z)
    bins = torch.cumsum(counts, 0).int().cuda()
    a = (torch.randn(rows, m) * 0.5).to(dtype).cuda()
    b = (torch.randn(rows, n) * 0.5).to(dtype).cuda()
    sink = G.GradNormSink(torch.device('cuda', 0), slots=8)
    sink.begin()
    G.set_grad_norm_sink(sink)
    try:
        first, _, _ = G.grouped_gemm(a, b, bins, trans_a=True, num_groups=z, alpha=0.5, grad_norm=True)
        unasked, _, _ = G.grouped_gemm(a, b, bins, trans_a=True, num_groups=z)               # no slot taken
        second, _, _ = G.grouped_gemm(b, a, bins, trans_a=True, num_groups=z, grad_norm=True)
    finally:
        G.set_grad_norm_sink(None)
    after, _, _ = G.grouped_gemm(a, b, bins, trans_a=True, num_groups=z, grad_norm=True)     # no sink: ignored
    assert sink.lookup(first) == 0 and sink.lookup(second) == 1
    assert sink.lookup(unasked) is None and sink.lookup(after) is None and sink.lookup(first[0]) is None
    got = sink.slots.cpu()
    for slot, out in ((0, first), (1, second)):
        want = float(out.float().square().sum())
        assert abs(float(got[slot]) - want) <= 4e-3 * want       # fp32 values before their rounding to bf16
    assert float(got[2:].abs().sum()) == 0.0
