"""Block-sparse Matrix products against dense matmuls."""

import pytest
import torch
from conftest import DEVICES

from megablocks_b200.ops import sparse


def _rand_sparse(rows, cols, sparsity, blocking, device):
    mask = sparse.random_mask(rows, cols, sparsity, blocking, dtype=torch.float32)
    vals = torch.randn(mask.data.shape)
    return sparse.with_data(mask, vals.to(device)), mask


def _to(m, device):
    out = sparse.Matrix(m.size(), m.data.to(device), m.row_indices.to(device), m.column_indices.to(device),
                        m.offsets.to(device), m.column_indices_t.to(device), m.offsets_t.to(device),
                        m.block_offsets_t.to(device))
    return out


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('m,k,n,blocking,sparsity', [(256, 128, 384, 128, 0.0), (256, 64, 512, 128, 0.5),
                                                     (64, 48, 96, 16, 0.6)])
def test_products(device, m, k, n, blocking, sparsity):
    topo, _ = _rand_sparse(m, n, sparsity, blocking, 'cpu')
    topo = _to(topo, device)
    dense_mask = (sparse.to_dense(sparse.with_data(topo, torch.ones_like(topo.data))) != 0).float()

    a = torch.randn(m, k, device=device, requires_grad=True)
    b = torch.randn(k, n, device=device, requires_grad=True)
    s = sparse.sdd(a, b, topo)
    ref = (a @ b) * dense_mask
    torch.testing.assert_close(sparse.to_dense(s), ref, rtol=1e-4, atol=1e-4)
    probe = torch.randn(m, n, device=device)
    ga, gb = torch.autograd.grad((sparse.to_dense(s) * probe).sum(), (a, b), retain_graph=True)
    ra, rb = torch.autograd.grad((ref * probe).sum(), (a, b), retain_graph=True)
    torch.testing.assert_close(ga, ra, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gb, rb, rtol=1e-4, atol=1e-4)

    data = topo.data.clone().requires_grad_(True)
    sm = sparse.with_data(topo, data)
    w = torch.randn(n, 40, device=device, requires_grad=True)
    out = sparse.dsd(sm, w)
    dense = sparse.to_dense(sm)
    torch.testing.assert_close(out, dense @ w, rtol=1e-4, atol=1e-4)
    g1 = torch.autograd.grad(out.sum(), (data, w), retain_graph=True)
    g2 = torch.autograd.grad((dense @ w).sum(), (data, w), retain_graph=True)
    for x, y in zip(g1, g2):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)

    v = torch.randn(m, 24, device=device, requires_grad=True)
    out_t = sparse.dsd(sm.t(), v)
    torch.testing.assert_close(out_t, dense.t() @ v, rtol=1e-4, atol=1e-4)
    g1 = torch.autograd.grad(out_t.sum(), (data, v), retain_graph=True)
    g2 = torch.autograd.grad((dense.t() @ v).sum(), (data, v), retain_graph=True)
    for x, y in zip(g1, g2):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)

    u = torch.randn(24, m, device=device, requires_grad=True)
    out_d = sparse.dds(u, sm)
    torch.testing.assert_close(out_d, u @ dense, rtol=1e-4, atol=1e-4)
    g1 = torch.autograd.grad(out_d.sum(), (u, data), retain_graph=True)
    g2 = torch.autograd.grad((u @ dense).sum(), (u, data), retain_graph=True)
    for x, y in zip(g1, g2):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(sparse.dds(w.t().contiguous()[:, :n], sm.t()), w.t()[:, :n] @ dense.t(), rtol=1e-4,
                               atol=1e-4)


def test_transpose_metadata_roundtrip():
    m, _ = _rand_sparse(512, 384, 0.4, 128, 'cpu')
    dense = sparse.to_dense(m)
    mt = sparse.to_sparse(dense.t().contiguous(), 128)
    # Blocks listed in transposed order must equal the transposed matrix's blocks.
    order = m.block_offsets_t.long()
    torch.testing.assert_close(m.data[order].transpose(1, 2), mt.data)
    assert torch.equal(m.column_indices_t.long(), mt.column_indices.long())
    assert torch.equal(m.offsets_t, mt.offsets)
    assert torch.equal(sparse.row_indices(m.size(), m.data, m.offsets, m.column_indices).long(),
                       m.row_indices.long())
    assert sparse.mul(m, m).data.equal(m.data * m.data)


def _launches():
    from megablocks_b200._ext import ext
    return ext().launch_count()


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('m,k,n,sparsity', [(256, 128, 384, 0.0), (512, 200, 640, 0.5), (1024, 64, 1280, 0.9),
                                            (128, 72, 128, 0.0), (768, 384, 512, 0.5)])
def test_tensor_core_products_match_fp32(m, k, n, sparsity, dtype):
    """sdd / dsd / dds on 128 x 128 blocks run the BCSR-driven tcgen05 kernel; oracle: dense fp32 matmuls.

    Covers plain and transposed dense operands, plain and transposed topologies, block rows and
    columns without any stored block, dense dimensions that are not multiples of the tile, and
    the autograd formulas (which use the transposed forms).
    """
    torch.manual_seed(m + n)
    dev = 'cuda'
    topo, _ = _rand_sparse(m, n, sparsity, 128, 'cpu')
    topo = sparse.with_data(_to(topo, dev), (torch.randn(topo.data.shape) * 0.5).to(dtype).to(dev))
    dense = sparse.to_dense(topo).float().cpu()
    mask = (sparse.to_dense(sparse.with_data(topo, torch.ones_like(topo.data))) != 0).float().cpu()

    def close(got, want):
        got, want = got.detach().float().cpu(), want.detach().float().cpu()
        torch.testing.assert_close(got, want, rtol=2e-2, atol=1e-2 * float(want.abs().max()) + 1e-3)

    a = (torch.randn(m, k) * 0.5).to(dtype).to(dev)
    b = (torch.randn(k, n) * 0.5).to(dtype).to(dev)
    before = _launches()
    # sdd with every combination of stored / transposed-view dense operands.
    want = (a.float().cpu() @ b.float().cpu()) * mask
    for av in (a, a.t().contiguous().t()):
        for bv in (b, b.t().contiguous().t()):
            close(sparse.to_dense(sparse.sdd(av, bv, topo)), want)
    assert _launches() - before >= 4, 'sdd did not run the tensor-core kernel'

    # dsd / dds, plain and transposed topology, odd dense widths.
    w = (torch.randn(n, 40) * 0.5).to(dtype).to(dev)
    v = (torch.randn(m, 24) * 0.5).to(dtype).to(dev)
    u = (torch.randn(24, m) * 0.5).to(dtype).to(dev)
    x = (torch.randn(200, n) * 0.5).to(dtype).to(dev)
    before = _launches()
    close(sparse.dsd(topo, w), dense @ w.float().cpu())
    close(sparse.dsd(topo, w.t().contiguous().t()), dense @ w.float().cpu())
    close(sparse.dsd(topo.t(), v), dense.t() @ v.float().cpu())
    close(sparse.dds(u, topo), u.float().cpu() @ dense)
    close(sparse.dds(u.t().contiguous().t(), topo), u.float().cpu() @ dense)
    close(sparse.dds(x, topo.t()), x.float().cpu() @ dense.t())
    assert _launches() - before >= 6, 'dsd / dds did not run the tensor-core kernel'

    # Autograd through all three (fp32 oracle through dense matmuls).
    a1 = a.clone().requires_grad_(True)
    b1 = b.clone().requires_grad_(True)
    a2 = a.float().cpu().requires_grad_(True)
    b2 = b.float().cpu().requires_grad_(True)
    probe = (torch.randn(m, n) * 0.5).to(dtype)
    (sparse.to_dense(sparse.sdd(a1, b1, topo)).float() * probe.to(dev).float()).sum().backward()
    (((a2 @ b2) * mask) * probe.float()).sum().backward()
    close(a1.grad, a2.grad)
    close(b1.grad, b2.grad)

    data = topo.data.clone().requires_grad_(True)
    sm = sparse.with_data(topo, data)
    w1 = w.clone().requires_grad_(True)
    d2 = dense.clone().requires_grad_(True)
    w2 = w.float().cpu().requires_grad_(True)
    pw = (torch.randn(m, 40) * 0.5).to(dtype)
    (sparse.dsd(sm, w1).float() * pw.to(dev).float()).sum().backward()
    ((d2 @ w2) * pw.float()).sum().backward()
    close(w1.grad, w2.grad)
    close(sparse.to_dense(sparse.with_data(topo, data.grad)), d2.grad * mask)

    data.grad = None
    u1 = u.clone().requires_grad_(True)
    d3 = dense.clone().requires_grad_(True)
    u2 = u.float().cpu().requires_grad_(True)
    pu = (torch.randn(24, n) * 0.5).to(dtype)
    (sparse.dds(u1, sm).float() * pu.to(dev).float()).sum().backward()
    ((u2 @ d3) * pu.float()).sum().backward()
    close(u1.grad, u2.grad)
    close(sparse.to_dense(sparse.with_data(topo, data.grad)), d3.grad * mask)

    data.grad = None
    v1 = v.clone().requires_grad_(True)
    d4 = dense.clone().requires_grad_(True)
    v2 = v.float().cpu().requires_grad_(True)
    pv = (torch.randn(n, 24) * 0.5).to(dtype)
    (sparse.dsd(sm.t(), v1).float() * pv.to(dev).float()).sum().backward()
    ((d4.t() @ v2) * pv.float()).sum().backward()
    close(v1.grad, v2.grad)
    close(sparse.to_dense(sparse.with_data(topo, data.grad)), d4.grad * mask)
    from megablocks_b200.utils import status
    status.check()
