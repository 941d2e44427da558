"""Randomised-shape fuzz of the routing / permutation / grouped-GEMM ops against CPU restatements,
with the debug range checks on, plus the range checks themselves and a double-run determinism check.

Stands in for a memory sanitizer (not available where this library is developed): every index a
kernel consumes is validated before the launch (``MB200_DEBUG_BOUNDS`` / ``utils.debug``), shapes
are drawn at random including empty experts, single tokens and odd widths, and every result is
compared with a plain PyTorch restatement of the op.
"""

import random

import pytest
import torch
from conftest import DEVICES

from megablocks_b200 import ops
from megablocks_b200.ops import gg as G
from megablocks_b200.utils import debug


@pytest.fixture(autouse=True)
def _bounds_on():
    debug.enable(True)
    yield
    debug.enable(False)


def _ref_gather(x, indices, bins, top_k):
    return x[indices.long() // top_k]


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('seed', range(12))
def test_fuzz_route_gather_gemm_scatter(device, seed):
    rng = random.Random(seed)
    tokens = rng.choice([1, 2, 7, 33, 128, 500, 1111])
    experts = rng.choice([1, 2, 3, 8, 17, 64])
    top_k = rng.choice([k for k in (1, 2, 4) if k <= experts])
    hidden = rng.choice([8, 24, 64, 136])
    ffn = rng.choice([64, 72, 128])
    dtype = torch.float32 if device == 'cpu' else torch.bfloat16
    g = torch.Generator().manual_seed(seed)
    # Skewed routing: some experts get nothing.
    probs = torch.rand(experts, generator=g)**3 + 1e-3
    top = torch.stack([torch.multinomial(probs, top_k, replacement=False, generator=g) for _ in range(tokens)])
    weights = torch.rand(tokens * top_k, generator=g).to(dtype).to(device)
    x = torch.randn(tokens, hidden, generator=g).to(dtype).to(device)
    top_dev = top.flatten().int().to(device)

    indices, bin_ids, bins, padded_bins, tpe = ops.route_plan(top_dev, experts, 128)
    # CPU restatement of the plan.
    flat = top.flatten().long()
    sorted_ids, order = torch.sort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    assert torch.equal(indices.cpu().long(), order) and torch.equal(bin_ids.cpu().long(), sorted_ids)
    assert torch.equal(tpe.cpu().long(), counts) and torch.equal(bins.cpu().long(), torch.cumsum(counts, 0))

    xg = ops.gather(x, indices, bin_ids, bins, top_k)
    torch.testing.assert_close(xg.cpu(), _ref_gather(x.cpu(), indices.cpu(), bins.cpu(), top_k))

    w = (torch.randn(experts, ffn, hidden, generator=g) * 0.2).to(dtype).to(device)
    y = G.gmm_bins(xg, w, bins, trans_b=True)
    ref = torch.zeros(tokens * top_k, ffn)
    start = 0
    for e, c in enumerate(counts.tolist()):
        ref[start:start + c] = xg[start:start + c].float().cpu() @ w[e].float().cpu().t()
        start += c
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2 * float(ref.abs().max()) + 1e-3)
    torch.testing.assert_close(y.float().cpu(), ref, **tol)

    out = ops.scatter(y, indices, bin_ids, weights, bins, top_k)
    back = torch.zeros(tokens, ffn)
    contrib = y.float().cpu() * weights.float().cpu()[indices.cpu().long()].unsqueeze(1)
    back.index_add_(0, indices.cpu().long() // top_k, contrib)
    torch.testing.assert_close(out.float().cpu(), back, **tol)

    # Same inputs, second run: bitwise identical (no floating-point atomics anywhere on this path).
    out2 = ops.scatter(G.gmm_bins(ops.gather(x, indices, bin_ids, bins, top_k), w, bins, trans_b=True), indices, bin_ids,
                       weights, bins, top_k)
    assert torch.equal(out, out2)

    # Padded forms.
    rows = int(padded_bins[-1]) if padded_bins.numel() else 0
    xp = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k, num_rows=rows + 128)
    outp = ops.padded_scatter(xp, indices, bin_ids, weights, bins, padded_bins, top_k)
    refp = torch.zeros(tokens, hidden)
    refp.index_add_(0, indices.cpu().long() // top_k,
                    _ref_gather(x.cpu(), indices.cpu(), bins.cpu(), top_k).float() *
                    weights.float().cpu()[indices.cpu().long()].unsqueeze(1))
    tolp = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(outp.float().cpu(), refp, **tolp)


@pytest.mark.parametrize('device', DEVICES)
def test_range_checks_refuse_bad_metadata(device):
    x = torch.randn(8, 16, device=device)
    top = torch.tensor([0, 1, 1, 0, 2, 2, 1, 0], dtype=torch.int32, device=device)
    indices, bin_ids, bins, padded_bins, _ = ops.route_plan(top, 3, 4)
    ops.gather(x, indices, bin_ids, bins, 1)                         # sane metadata passes
    bad = indices.clone()
    bad[3] = 99                                                      # a copy id that does not exist
    with pytest.raises(debug.BoundsError, match='indices'):
        ops.gather(x, bad, bin_ids, bins, 1)
    bad_bins = bins.clone()
    bad_bins[1] = 1                                                  # decreasing prefix sum
    with pytest.raises(debug.BoundsError, match='bins'):
        ops.gather(x, indices, bin_ids, bad_bins, 1)
    with pytest.raises(debug.BoundsError, match='padded_bins'):
        ops.padded_gather(x, indices, bin_ids, bins, padded_bins, 1, num_rows=4)   # output too small
    with pytest.raises(debug.BoundsError, match='bins'):
        G.gmm_bins(x, torch.randn(3, 16, 16, device=device), torch.tensor([4, 9, 12], dtype=torch.int32,
                                                                          device=device))
    debug.enable(False)
    assert not debug.enabled()
