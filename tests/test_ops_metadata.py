"""sort / histogram / cumsum / round_up / topology / replicate against inline oracles.

Case lists follow the reference op tests (tests/ops/sort_test.py:12-65,
histogram_test.py:9-82, cumsum_test.py:9-44, topology_test.py:10-81,
replicate_test.py:20-108).
"""

import numpy as np
import pytest
import torch
from conftest import DEVICES

from megablocks_b200 import ops

INT_DTYPES = [torch.int16, torch.int32, torch.int64]


def _max_for(dtype, limit):
    return min(limit, torch.iinfo(dtype).max) if limit else torch.iinfo(dtype).max


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('n', [32, 1024, 16384, 1000])
@pytest.mark.parametrize('dtype', INT_DTYPES)
@pytest.mark.parametrize('limit', [None, 128])
def test_sort(device, n, dtype, limit):
    hi = _max_for(dtype, limit)
    end_bit = None if limit is None else int(np.ceil(np.log2(hi)))
    x = torch.randint(0, hi, (n,), dtype=torch.int64).to(dtype).to(device)
    keys, perm = ops.sort(x, end_bit)
    assert perm.dtype == dtype and keys.dtype == dtype
    expected, _ = torch.sort(x.cpu())
    assert torch.equal(keys.cpu(), expected)
    # The permutation must reproduce the keys and be a bijection.
    assert torch.equal(x.cpu()[perm.cpu().long()], expected)
    if n <= torch.iinfo(dtype).max:
        assert torch.equal(torch.sort(perm.cpu().long())[0], torch.arange(n))


@pytest.mark.parametrize('device', DEVICES)
def test_sort_is_stable(device):
    x = torch.randint(0, 4, (4096,), dtype=torch.int32, device=device)
    _, perm = ops.sort(x, 2)
    expected = torch.argsort(x.cpu(), stable=True)
    assert torch.equal(perm.cpu().long(), expected)


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('batch', [1, 2, 8])
@pytest.mark.parametrize('n', [32, 1024, 16384])
@pytest.mark.parametrize('dtype', INT_DTYPES)
@pytest.mark.parametrize('bins', [2, 128, 1024])
def test_histogram(device, batch, n, dtype, bins):
    x = torch.randint(0, bins, (batch, n), dtype=torch.int64).to(dtype).to(device)
    out = ops.histogram(x, bins)
    assert out.dtype == torch.int32 and out.shape == (batch, bins)
    for b in range(batch):
        assert torch.equal(out[b].cpu().long(), torch.bincount(x[b].cpu().long(), minlength=bins))
    flat = ops.histogram(x[0], bins)
    assert flat.shape == (bins,) and torch.equal(flat, out[0])


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('shape', [(1, 32), (2, 1024), (16, 128), (128, 16384), (3, 1), (1, 1)])
@pytest.mark.parametrize('dtype', INT_DTYPES)
def test_cumsum(device, shape, dtype):
    x = torch.randint(0, 2, shape, dtype=torch.int64).to(dtype).to(device)
    inc = ops.inclusive_cumsum(x, 1)
    exc = ops.exclusive_cumsum(x, 1)
    ref = torch.cumsum(x.cpu().long(), dim=1)
    assert torch.equal(inc.cpu().long(), ref)
    assert torch.equal(exc.cpu().long(), ref - x.cpu().long())
    assert inc.dtype == dtype


@pytest.mark.parametrize('device', DEVICES)
def test_cumsum_1d_squeeze_quirk(device):
    one = torch.tensor([5], dtype=torch.int32, device=device)
    assert ops.inclusive_cumsum(one, 0).dim() == 0
    many = torch.tensor([1, 2, 3], dtype=torch.int32, device=device)
    assert ops.inclusive_cumsum(many, 0).tolist() == [1, 3, 6]
    assert ops.exclusive_cumsum(many, 0).tolist() == [0, 1, 3]


@pytest.mark.parametrize('device', DEVICES)
def test_round_up(device):
    x = torch.tensor([0, 1, 127, 128, 129, 1000], dtype=torch.int32, device=device)
    assert ops.round_up(x, 128).tolist() == [0, 128, 128, 128, 256, 1024]


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('sl,hs,ne', [(1024, 1536, 2), (1024, 1536, 4), (1024, 1536, 8), (1024, 1536, 16),
                                       (1024, 1536, 32), (1024, 1536, 64), (1024, 1536, 128), (16384, 768, 128),
                                       (16384, 768, 1024), (8, 14336, 8), (1024, 128, 3)])
def test_topology(device, sl, hs, ne):
    blocking = 128
    assert hs % blocking == 0
    top_expert = torch.randint(0, ne, (sl,), dtype=torch.int32)
    tpe = torch.bincount(top_expert.long(), minlength=ne).int()
    padded = ((tpe + blocking - 1) // blocking) * blocking
    padded_bins = torch.cumsum(padded, 0).int()
    block_rows = int(padded_bins[-1]) // blocking
    cols = hs // blocking
    out = ops.topology(padded_bins.to(device), blocking, block_rows, cols)
    assert out.dtype == torch.int16
    expected = []
    for e in range(ne):
        for _ in range(int(padded[e]) // blocking):
            expected.extend(range(e * cols, (e + 1) * cols))
    assert out.cpu().tolist() == [np.int16(v).item() for v in np.asarray(expected, dtype=np.int64).astype(np.int16)]


@pytest.mark.parametrize('device', DEVICES)
@pytest.mark.parametrize('tokens', [8, 1024, 16384])
@pytest.mark.parametrize('num_centers', [1, 4, 128])
@pytest.mark.parametrize('top_k', [1, 4, 8])
@pytest.mark.parametrize('dtype', [torch.float16, torch.int32, torch.float32])
def test_replicate(device, tokens, num_centers, top_k, dtype):
    tokens_per_center = torch.bincount(torch.randint(0, num_centers, (tokens,)), minlength=num_centers)
    bins = torch.cumsum(tokens_per_center, 0).int().to(device)
    if dtype.is_floating_point:
        x = torch.randn(top_k, num_centers).to(dtype)
    else:
        x = torch.randint(0, 1000, (top_k, num_centers), dtype=dtype)
    x = x.to(device)
    if dtype.is_floating_point:
        x.requires_grad_(True)
    out = ops.replicate(x, bins, tokens)
    expected = torch.repeat_interleave(x.detach().cpu(), tokens_per_center, dim=1)
    assert torch.equal(out.detach().cpu(), expected)
    if dtype.is_floating_point:
        out.backward(torch.ones_like(out))
        ref = (tokens_per_center.to(torch.float32).unsqueeze(0).expand(top_k, -1))
        torch.testing.assert_close(x.grad.cpu().float(), ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize('device', DEVICES)
def test_repeat_and_sum(device):
    x = torch.arange(6, device=device).view(2, 3)
    assert ops.repeat(x, (1, 1)) is x
    assert ops.repeat(x, (2, 1)).shape == (4, 3)
    assert ops.sum(x.view(1, 2, 3), dim=0).shape == (2, 3)
    assert torch.equal(ops.sum(x, dim=0), x.sum(0))


def test_micro_benchmark_scripts_run_on_the_host():
    """The sort / histogram / padded-scatter benchmark entry points (the reference ships one file each)."""
    from megablocks_b200.benchmarks import histogram_benchmark, padded_scatter_benchmark, sort_benchmark
    cpu = torch.device('cpu')
    rows = sort_benchmark.run(cpu, iters=1)
    assert len(rows) == len(sort_benchmark.SORT_CASES) and all(r['ops.sort_us'] > 0 for r in rows)
    rows = histogram_benchmark.run(cpu, iters=1)
    assert [r['bins'] for r in rows] == [2, 4, 8, 16, 32, 64, 128, 256]
    rows = padded_scatter_benchmark.run(cpu, iters=1, cases=((512, 64, 8, 4), (2048, 64, 8, 1)))
    assert len(rows) == 2 and all(r['forward_us'] > 0 and r['backward_us'] > 0 for r in rows)
