"""The allocation-free route plan, called through its exported C symbol.

``mb_route_plan_noalloc`` serves callers that cannot allocate device memory (code
living inside another runtime's arena, engines with a frozen memory map, sandboxes
that deny cudaMalloc): they bring every buffer and the library's own fixed scratch
array does the rest.  The test calls the symbol with ctypes exactly as such a caller
would, twice in a row with different inputs (the scratch keeps the first call's
contents), and requires bit-equal results with the regular ``route_plan`` op and with a
plain CPU oracle (stable sort, bincount, cumsum), which shares no kernel with either.  It
also checks that oversize requests are refused before anything is launched.

This file sorts last on purpose: if it ever fails, a run that stops at the first
failure has already executed every other test.
"""

import ctypes

import pytest
import torch

CUDA_ERROR_INVALID_VALUE = 1


def _symbol():
    from megablocks_b200._ext import ext
    lib = ctypes.CDLL(ext().__file__)
    fn = lib.mb_route_plan_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


@pytest.mark.gpu
def test_route_plan_noalloc_matches_route_plan_twice_in_a_row():
    from megablocks_b200 import ops
    fn = _symbol()
    dev = torch.device('cuda', 0)
    stream = torch.cuda.current_stream(dev)
    for n, experts, block, seed in [(32768, 64, 128, 1), (100000, 1000, 128, 2), (7, 3, 16, 3)]:
        gen = torch.Generator(device='cpu').manual_seed(seed)
        top = torch.randint(0, experts, (n,), generator=gen, dtype=torch.int32).to(dev)
        # The caller's buffers: allocated up front, before the calls under test.
        indices = torch.full((n,), -1, dtype=torch.int32, device=dev)
        bin_ids = torch.full((n,), -1, dtype=torch.int32, device=dev)
        bins = torch.full((experts,), -1, dtype=torch.int32, device=dev)
        padded = torch.full((experts,), -1, dtype=torch.int32, device=dev)
        tpe = torch.full((experts,), -1, dtype=torch.int32, device=dev)
        rc = fn(top.data_ptr(), n, experts, block, indices.data_ptr(), bin_ids.data_ptr(), bins.data_ptr(),
                padded.data_ptr(), tpe.data_ptr(), stream.cuda_stream)
        assert rc == 0
        want = ops.route_plan(top, experts, block)
        torch.cuda.synchronize()
        for got, ref in zip((indices, bin_ids, bins, padded, tpe), want):
            assert torch.equal(got, ref)
        # Independent oracle on the host.
        host = top.cpu().long()
        sorted_ids, order = torch.sort(host, stable=True)
        counts = torch.bincount(host, minlength=experts)
        assert torch.equal(indices.cpu().long(), order)
        assert torch.equal(bin_ids.cpu().long(), sorted_ids)
        assert torch.equal(tpe.cpu().long(), counts)
        assert torch.equal(bins.cpu().long(), torch.cumsum(counts, 0))
        assert torch.equal(padded.cpu().long(), torch.cumsum((counts + block - 1) // block * block, 0))


@pytest.mark.gpu
def test_route_plan_noalloc_rejects_sizes_beyond_the_maximum():
    fn = _symbol()
    dev = torch.device('cuda', 0)
    buf = torch.zeros(16, dtype=torch.int32, device=dev)
    p = buf.data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert fn(p, (1 << 20) + 1, 8, 128, p, p, p, p, p, stream) == CUDA_ERROR_INVALID_VALUE
    assert fn(p, 16, 1025, 128, p, p, p, p, p, stream) == CUDA_ERROR_INVALID_VALUE
    assert fn(p, 16, 8, 0, p, p, p, p, p, stream) == CUDA_ERROR_INVALID_VALUE
    torch.cuda.synchronize()
