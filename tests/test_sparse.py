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
