"""Padded scatter benchmark on the reference's two shapes (megablocks/ops/padded_scatter_benchmark.py:11-16:
dMoE-Medium with 8-way expert parallelism before and after the all-to-all), forward and backward.

    python -m megablocks_b200.benchmarks.padded_scatter_benchmark [--iters N] [--device cuda|cpu]
"""

import argparse

import torch

from megablocks_b200 import ops
from megablocks_b200.benchmark_util import benchmark_function

PADDED_SCATTER_CASES = ((1024 * 16, 1024, 8, 4), (1024 * 16 * 4, 1024, 8, 1))


def run(device: torch.device, iters: int, cases=PADDED_SCATTER_CASES):
    rows = []
    dtype = torch.bfloat16 if device.type == 'cuda' else torch.float32
    for sl, hs, ne, top_k in cases:
        top = torch.randint(0, ne, (sl * top_k,), dtype=torch.int32).to(device)
        indices, bin_ids, bins, padded_bins, _ = ops.route_plan(top, ne)
        x = torch.randn(sl, hs, dtype=dtype).to(device)
        w = torch.rand(sl * top_k, dtype=dtype).to(device).requires_grad_(True)
        gathered = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k).detach().requires_grad_(True)

        def forward():
            return ops.padded_scatter(gathered, indices, bin_ids, w, bins, padded_bins, top_k)

        out = forward()
        grad = torch.randn_like(out)

        def backward():
            gathered.grad = w.grad = None
            out.backward(grad, retain_graph=True)

        fwd, _ = benchmark_function(forward, iterations=iters, warmup=3)
        bwd, _ = benchmark_function(backward, iterations=iters, warmup=3)
        moved = 2.0 * sl * top_k * hs * x.element_size()
        rows.append({'tokens': sl, 'hidden': hs, 'experts': ne, 'top_k': top_k, 'forward_us': fwd * 1e3,
                     'backward_us': bwd * 1e3, 'forward_GBs': moved / fwd / 1e6})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--device', default='cuda' if torch.cuda.is_available() else 'cpu')
    args = ap.parse_args()
    for row in run(torch.device(args.device), args.iters):
        print('  '.join(f'{k}={v:.1f}' if isinstance(v, float) else f'{k}={v}' for k, v in row.items()))


if __name__ == '__main__':
    main()
