"""``grouped_gemm.backend.gmm``: per-group cuBLAS matmuls (the package's non-CUTLASS mode)."""

import torch


def gmm(a, b, batch_sizes, trans_a=False, trans_b=False, c=None):
    sizes = batch_sizes.tolist()
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
