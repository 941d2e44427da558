"""Permutation / metadata benchmark: gather, scatter, padded and binned forms, sort, histogram, route plan.

Shapes follow megablocks/ops/permute_benchmark.py:11-26, padded_scatter_benchmark.py:11-16,
sort_benchmark.py:12-16 and histogram_benchmark.py:12-21 of the reference.  Reports
milliseconds and achieved bandwidth against the measured copy bandwidth.

    python -m megablocks_b200.benchmarks.permute_benchmark [--iters N]
"""

import argparse
import json
import os

import torch

from megablocks_b200 import ops
from megablocks_b200.benchmark_util import benchmark_function

PERMUTE = [(16384, 768, e, 1) for e in (2, 8, 64, 128)] + [(131072, 768, 64, 1), (16384, 1024, 8, 4),
                                                             (65536, 1024, 8, 1), (32768, 768, 64, 1)]


def measured_hbm_gbs():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--iters', type=int, default=20)
    args = ap.parse_args()
    dev = torch.device('cuda')
    peak, kind = measured_hbm_gbs()
    for sl, hs, ne, top_k in PERMUTE:
        x = torch.randn(sl, hs, device=dev, dtype=torch.bfloat16)
        top = torch.randint(0, ne, (sl * top_k,), device=dev, dtype=torch.int32)
        w = torch.rand(sl * top_k, device=dev, dtype=torch.bfloat16)
        indices, bin_ids, bins, padded_bins, tpe = ops.route_plan(top, ne)
        g = ops.gather(x, indices, bin_ids, bins, top_k)
        pg = ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k)
        cap = sl * top_k // ne
        bg = ops.binned_gather(x, indices, bins, cap, top_k)
        moved = 2.0 * sl * top_k * hs * 2
        cases = {
            'route_plan': (lambda: ops.route_plan(top, ne), None),
            'gather': (lambda: ops.gather(x, indices, bin_ids, bins, top_k), moved),
            'scatter': (lambda: ops.scatter(g, indices, bin_ids, w, bins, top_k), moved),
            'padded_gather': (lambda: ops.padded_gather(x, indices, bin_ids, bins, padded_bins, top_k,
                                                        num_rows=pg.shape[0]), moved),
            'padded_scatter': (lambda: ops.padded_scatter(pg, indices, bin_ids, w, bins, padded_bins, top_k), moved),
            'binned_gather': (lambda: ops.binned_gather(x, indices, bins, cap, top_k), moved),
            'binned_scatter': (lambda: ops.binned_scatter(bg, indices, w, bins, top_k), moved),
        }
        print(f'tokens={sl} hidden={hs} experts={ne} top_k={top_k}')
        for name, (fn, nbytes) in cases.items():
            mean, std = benchmark_function(fn, iterations=args.iters, warmup=5, flush_l2=True)
            bw = '' if nbytes is None else f'{nbytes / mean / 1e6:8.0f} GB/s  {nbytes / mean / 1e6 / peak:5.2f} of {kind} copy bandwidth'
            print(f'  {name:16s} {mean * 1e3:9.1f} us +- {std * 1e3:6.1f}  {bw}')
    for n in (16384, 131072):
        for dtype in (torch.int16, torch.int32, torch.int64):
            keys = torch.randint(0, 128, (n,), device=dev).to(dtype)
            mean, std = benchmark_function(lambda: ops.sort(keys, 7), iterations=args.iters, warmup=5)
            print(f'sort n={n} {dtype}: {mean * 1e3:.1f} us')
            mean, std = benchmark_function(lambda: ops.histogram(keys, 128), iterations=args.iters, warmup=5)
            print(f'histogram n={n} {dtype}: {mean * 1e3:.1f} us')


if __name__ == '__main__':
    main()
