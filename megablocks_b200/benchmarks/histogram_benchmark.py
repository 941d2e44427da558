"""Histogram benchmark: ``ops.histogram`` against ``torch.histc`` on the reference's cases
(megablocks/ops/histogram_benchmark.py:12-21: 16384 int32 values in 2 .. 256 bins).

    python -m megablocks_b200.benchmarks.histogram_benchmark [--iters N] [--device cuda|cpu]
"""

import argparse

import torch

from megablocks_b200 import ops
from megablocks_b200.benchmark_util import benchmark_function

HISTOGRAM_CASES = tuple((16384, torch.int32, bins) for bins in (2, 4, 8, 16, 32, 64, 128, 256))


def run(device: torch.device, iters: int):
    rows = []
    for n, dtype, bins in HISTOGRAM_CASES:
        x = torch.randint(0, bins, (n,), dtype=dtype).to(device)
        xf = x.float()
        ours, _ = benchmark_function(lambda: ops.histogram(x, bins), iterations=iters, warmup=3)
        base, _ = benchmark_function(lambda: torch.histc(xf, bins, 0, bins - 1), iterations=iters, warmup=3)
        rows.append({'n': n, 'bins': bins, 'ops.histogram_us': ours * 1e3, 'torch.histc_us': base * 1e3})
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
