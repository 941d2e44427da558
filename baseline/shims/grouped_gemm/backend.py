"""``grouped_gemm.backend.gmm`` stand-in with two modes.

``MB_REF_GMM=loop`` (default): one library (cuBLAS) matmul per expert over row counts held on the
host - the package's default, non-CUTLASS build.  ``MB_REF_GMM=grouped_mm``: one
``torch._grouped_mm`` launch per call, the analogue of the package's ``GROUPED_GEMM_CUTLASS=1``
build that the reference's README recommends.  Selected by ``bench.py --ref-gmm``.
"""

import os

import torch

MODE = os.environ.get('MB_REF_GMM', 'loop')


def _loop(a, b, sizes, trans_a, trans_b, c):
    if trans_a:
        out = c if c is not None else a.new_empty(len(sizes), a.shape[1], b.shape[1])
        start = 0
        for e, n in enumerate(sizes):
            torch.matmul(a[start:start + n].t(), b[start:start + n], out=out[e])
            start += n
        return out
    n_out = b.shape[1] if trans_b else b.shape[2]
    out = c if c is not None else a.new_empty(a.shape[0], n_out)
    start = 0
    for e, n in enumerate(sizes):
        rhs = b[e].t() if trans_b else b[e]
        torch.matmul(a[start:start + n], rhs, out=out[start:start + n])
        start += n
    return out


def _grouped_mm(a, b, batch_sizes, trans_a, trans_b, c):
    offs = torch.cumsum(batch_sizes, 0).to(dtype=torch.int32).to(a.device, non_blocking=True)
    if trans_a:
        # [E, M, N] = a[rows of e]^T b[rows of e]: contraction over the ragged dimension.
        out = torch._grouped_mm(a.t(), b, offs=offs)
    else:
        out = torch._grouped_mm(a, b.transpose(1, 2) if trans_b else b, offs=offs)
    if c is not None:
        c.copy_(out)
        return c
    return out


def gmm(a, b, batch_sizes, trans_a=False, trans_b=False, c=None):
    if MODE == 'grouped_mm':
        return _grouped_mm(a, b, batch_sizes, trans_a, trans_b, c)
    return _loop(a, b, batch_sizes.tolist(), trans_a, trans_b, c)
