"""gather / scatter (+ padded, binned) forward and backward against Python-loop oracles.

Case lists follow tests/ops/padded_gather_test.py:10-94, padded_scatter_test.py:10-155,
binned_gather_test.py:10-71 and binned_scatter_test.py:10-87 of the reference; the
unpadded ops and the weight-gradient kernels, which the reference only covers through
layer tests, are tested directly here.
"""

import pytest
import torch
from conftest import DEVICES

from megablocks_b200 import ops

CASES = [
    (4, 2, 2, 1), (4, 2, 2, 2), (4, 2, 2, 4),
    (1024, 1, 4, 1), (1024, 1, 4, 2), (1024, 1, 64, 4), (1024, 1, 128, 1),
    (1024, 1536, 4, 1), (1024, 1536, 4, 2), (1024, 1536, 64, 4), (1024, 1536, 128, 2),
    (4096, 768, 64, 1), (4096, 768, 128, 4), (1000, 520, 7, 3),
]


def _route(sl, ne, top_k, device, blocking=128):
    top_expert = torch.randint(0, ne, (sl * top_k,), dtype=torch.int32, device=device)
    indices, bin_ids, bins, padded_bins, tpe = ops.route_plan(top_expert, ne, blocking)
    return top_expert, indices, bin_ids, bins, padded_bins, tpe


def _loop_gather(x, indices, bin_ids, bins, padded_bins, top_k, rows):
    out = torch.zeros(rows, x.shape[1], dtype=x.dtype)
    n = indices.numel()
    in_idx = 0
    for e in range(bins.numel()):
        end = int(bins[e])
        out_idx = 0 if e == 0 else int(padded_bins[e - 1])
        while in_idx < end:
            out[out_idx] = x[int(indices[in_idx]) // top_k]
            in_idx += 1
            out_idx += 1
    assert in_idx == n
    return out


def _loop_scatter(x, indices, bin_ids, weights, bins, padded_bins, top_k):
    tokens = indices.numel() // top_k
    out = torch.zeros(tokens * top_k, x.shape[1], dtype=torch.float32)
    in_idx = 0
    for e in range(bins.numel()):
        end = int(bins[e])
        src = 0 if e == 0 else int(padded_bins[e - 1])
        while in_idx < end:
            c = int(indices[in_idx])
            scale = float(weights[c]) if weights is not None else 1.0
            out[c] = x[src].float() * scale
            in_idx += 1
            src += 1
    return out.view(tokens, top_k, -1).sum(1)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('sl,hs,ne,top_k', CASES)
@pytest.mark.parametrize('padded', [False, True])
def test_gather_scatter(device, sl, hs, ne, top_k, padded):
    dtype = torch.float16
    x = torch.randn(sl, hs).to(dtype).to(device)
    _, indices, bin_ids, bins, padded_bins, _ = _route(sl, ne, top_k, device)
    pb = padded_bins if padded else bins
    if padded:
        out = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k)
    else:
        out = ops.gather(x, indices, bin_ids, bins, top_k)
    rows = int(pb[-1])
    expected = _loop_gather(x.cpu(), indices.cpu(), bin_ids.cpu(), bins.cpu(), pb.cpu(), top_k, rows)
    assert out.shape == expected.shape
    assert torch.equal(out.cpu(), expected)

    weights = torch.rand(sl * top_k).to(dtype).to(device)
    if padded:
        back = ops.padded_scatter(out, indices, bin_ids, weights, bins, padded_bins, top_k)
    else:
        back = ops.scatter(out, indices, bin_ids, weights, bins, top_k)
    ref = _loop_scatter(out.cpu(), indices.cpu(), bin_ids.cpu(), weights.cpu(), bins.cpu(), pb.cpu(), top_k)
    torch.testing.assert_close(back.cpu().float(), ref, rtol=5e-3, atol=5e-3)

    # Upper-bound sized padded buffer: rows past the last bin are zero.
    if padded:
        big = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k, num_rows=rows + 256)
        assert torch.equal(big[:rows].cpu(), expected) and not big[rows:].any()


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('sl,hs,ne,top_k', [(4, 2, 2, 2), (1024, 96, 8, 2), (512, 768, 64, 4), (256, 520, 5, 1)])
@pytest.mark.parametrize('padded', [False, True])
def test_scatter_backward(device, sl, hs, ne, top_k, padded):
    """dgrad and weight-grad of scatter, and dgrad of gather, against autograd on index ops."""
    x = torch.randn(sl, hs, device=device, dtype=torch.float32, requires_grad=True)
    w = torch.rand(sl * top_k, device=device, dtype=torch.float32, requires_grad=True)
    _, indices, bin_ids, bins, padded_bins, _ = _route(sl, ne, top_k, device)
    if padded:
        g = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k)
        y = ops.padded_scatter(g * 1.5, indices, bin_ids, w, bins, padded_bins, top_k)
    else:
        g = ops.gather(x, indices, bin_ids, bins, top_k)
        y = ops.scatter(g * 1.5, indices, bin_ids, w, bins, top_k)
    probe = torch.randn_like(y)
    (y * probe).sum().backward()

    x2 = x.detach().cpu().clone().requires_grad_(True)
    w2 = w.detach().cpu().clone().requires_grad_(True)
    y2 = (1.5 * x2.unsqueeze(1) * w2.view(sl, top_k, 1)).sum(1)
    (y2 * probe.cpu()).sum().backward()
    torch.testing.assert_close(y.detach().cpu(), y2.detach(), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x.grad.cpu(), x2.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(w.grad.cpu(), w2.grad, rtol=1e-3, atol=1e-3)


BINNED = [(4, 2, 2, 1), (4, 2, 2, 2), (4, 2, 2, 4), (1024, 1536, 4, 1), (1024, 1536, 64, 2), (1024, 1536, 128, 4),
          (4096, 768, 64, 1), (4096, 768, 128, 4)]


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('sl,hs,ne,top_k', BINNED)
def test_binned(device, sl, hs, ne, top_k):
    dtype = torch.float16
    capacity = (sl * top_k) // ne
    x = torch.randn(sl, hs).to(dtype).to(device)
    _, indices, _, bins, _, _ = _route(sl, ne, top_k, device)
    out = ops.binned_gather(x, indices, bins, capacity, top_k)
    assert out.shape == (ne, capacity, hs)

    xc, ic, bc = x.cpu(), indices.cpu(), bins.cpu()
    expected = torch.zeros(ne, capacity, hs, dtype=dtype)
    for e in range(ne):
        start = 0 if e == 0 else int(bc[e - 1])
        for j in range(min(capacity, int(bc[e]) - start)):
            expected[e, j] = xc[int(ic[start + j]) // top_k]
    assert torch.equal(out.cpu(), expected)

    weights = torch.rand(sl * top_k).to(dtype).to(device)
    back = ops.binned_scatter(out, indices, weights, bins, top_k)
    ref = torch.zeros(sl * top_k, hs)
    wc = weights.cpu().float()
    for e in range(ne):
        start = 0 if e == 0 else int(bc[e - 1])
        for j in range(min(capacity, int(bc[e]) - start)):
            c = int(ic[start + j])
            ref[c] = expected[e, j].float() * wc[c]
    ref = ref.view(sl, top_k, hs).sum(1)
    torch.testing.assert_close(back.cpu().float(), ref, rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize('device', DEVICES)
def test_binned_backward(device):
    sl, hs, ne, top_k = 256, 64, 8, 2
    capacity = 40  # forces drops for the busiest experts
    x = torch.randn(sl, hs, device=device, requires_grad=True)
    w = torch.rand(sl * top_k, device=device, requires_grad=True)
    _, indices, _, bins, _, _ = _route(sl, ne, top_k, device)
    y = ops.binned_scatter(ops.binned_gather(x, indices, bins, capacity, top_k), indices, w, bins, top_k)
    probe = torch.randn_like(y)
    (y * probe).sum().backward()

    # Oracle: mask of kept copies.
    ic, bc = indices.cpu().long(), bins.cpu().long()
    keep = torch.zeros(sl * top_k)
    for e in range(ne):
        start = 0 if e == 0 else int(bc[e - 1])
        keep[ic[start:start + min(capacity, int(bc[e]) - start)]] = 1
    x2 = x.detach().cpu().clone().requires_grad_(True)
    w2 = w.detach().cpu().clone().requires_grad_(True)
    y2 = (x2.unsqueeze(1) * (w2 * keep).view(sl, top_k, 1)).sum(1)
    (y2 * probe.cpu()).sum().backward()
    torch.testing.assert_close(y.detach().cpu(), y2.detach(), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x.grad.cpu(), x2.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(w.grad.cpu(), w2.grad, rtol=1e-3, atol=1e-3)
