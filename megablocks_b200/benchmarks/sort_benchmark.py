"""Sort benchmark: ``ops.sort`` against ``torch.sort`` on the reference's cases
(megablocks/ops/sort_benchmark.py:12-20: 16384 int32 keys, unbounded / 2 / 128 distinct values), plus
the route plan, which is what the layers call instead of a bare sort.

    python -m megablocks_b200.benchmarks.sort_benchmark [--iters N] [--device cuda|cpu]
"""

import argparse
import math

import torch

from megablocks_b200 import ops
from megablocks_b200.benchmark_util import benchmark_function

SORT_CASES = ((16384, torch.int32, None), (16384, torch.int32, 2), (16384, torch.int32, 128),
              (131072, torch.int32, 64))


def run(device: torch.device, iters: int):
    rows = []
    for n, dtype, max_val in SORT_CASES:
        hi = max_val if max_val is not None else torch.iinfo(dtype).max
        keys = torch.randint(0, hi, (n,), dtype=dtype).to(device)
        end_bit = None if max_val is None else max(1, math.ceil(math.log2(max_val)))
        ours, _ = benchmark_function(lambda: ops.sort(keys, end_bit), iterations=iters, warmup=3)
        base, _ = benchmark_function(lambda: torch.sort(keys), iterations=iters, warmup=3)
        row = {'n': n, 'max': max_val, 'ops.sort_us': ours * 1e3, 'torch.sort_us': base * 1e3}
        if max_val is not None:
            plan, _ = benchmark_function(lambda: ops.route_plan(keys, max_val), iterations=iters, warmup=3)
            row['route_plan_us'] = plan * 1e3
        rows.append(row)
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
