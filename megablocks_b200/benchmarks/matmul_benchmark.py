"""Expert GEMM benchmark: grouped NT / NN / TN products and the fused-epilogue forms.

Shapes ``(tokens, hidden, ffn, experts)`` follow the reference benchmark
(megablocks/ops/matmul_benchmark.py:24-29) plus the two models of the headline
configurations.  Reports milliseconds, TFLOP/s and the fraction of the measured
dense bf16 peak (``MEASURED_PEAKS.json`` at the repository root when present).

    python -m megablocks_b200.benchmarks.matmul_benchmark [--shape T H F E] [--iters N] [--zipf S]
                                                          [--case PREFIX] [--warmup N] [--pair 0|1]
"""

import argparse
import json
import os

import torch

from megablocks_b200.benchmark_util import benchmark_function
from megablocks_b200.ops import gg as G

SHAPES = (
    (65536, 512, 2048, 64),
    (32768, 768, 3072, 64),
    (8192, 1024, 4096, 64),
    (8192, 4096, 16384, 4),
    (16384, 1024, 4096, 64),
    (32768, 4096, 14336, 8),
)


def measured_peak_tflops():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)['bf16_tflops']), 'measured'
    return 1590.0, 'fallback'


def routed_bins(tokens, experts, zipf, device):
    if zipf > 0:
        p = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64)**zipf
        idx = torch.multinomial(p / p.sum(), tokens, replacement=True)
    else:
        idx = torch.randint(0, experts, (tokens,))
    counts = torch.bincount(idx, minlength=experts)
    return torch.cumsum(counts, 0).to(torch.int32).to(device)


def run_shape(tokens, hidden, ffn, experts, iters, zipf, dtype=torch.bfloat16, only=None, warmup=5, pair=None):
    dev = torch.device('cuda')
    peak, kind = measured_peak_tflops()
    bins = routed_bins(tokens, experts, zipf, dev)
    x = torch.randn(tokens, hidden, device=dev, dtype=dtype)
    h = torch.randn(tokens, ffn, device=dev, dtype=dtype)
    w = torch.randn(experts, ffn, hidden, device=dev, dtype=dtype) * 0.02
    flops = 2.0 * tokens * hidden * ffn
    cases = {
        'NT  x @ w1^T': lambda: G.grouped_gemm(x, w, bins, trans_b=True, pair=pair),
        'NT  + gelu epilogue (2 outputs)': lambda: G.grouped_gemm(x, w, bins, trans_b=True, epilogue=G.EPI_ACT,
                                                                  act=G.ACT_GELU_TANH, pair=pair),
        'NT  + gelu-backward epilogue': lambda: G.grouped_gemm(x, w, bins, trans_b=True, epilogue=G.EPI_DACT,
                                                               act=G.ACT_GELU_TANH, aux1=h, pair=pair),
        'NN  h @ w2': lambda: G.grouped_gemm(h, w, bins, pair=pair),
        'TN  h^T @ x (weight grad)': lambda: G.grouped_gemm(h, x, bins, trans_a=True, num_groups=experts, pair=pair),
    }
    print(f'shape tokens={tokens} hidden={hidden} ffn={ffn} experts={experts} zipf={zipf} pair={pair}')
    for name, fn in cases.items():
        if only is not None and not name.startswith(only):
            continue
        mean, std = benchmark_function(fn, iterations=iters, warmup=warmup, flush_l2=True)
        tf = flops / mean / 1e9
        print(f'  {name:34s} {mean:8.3f} ms +- {std:5.3f}  {tf:8.1f} TFLOP/s  {tf / peak:5.2f} of {kind} bf16 peak')


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--shape', type=int, nargs=4, metavar=('TOKENS', 'HIDDEN', 'FFN', 'EXPERTS'))
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--zipf', type=float, default=0.0)
    ap.add_argument('--case', type=str, default=None, help='run only the cases whose name starts with this')
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--pair', type=int, default=None, choices=(0, 1),
                    help='force the single-CTA (0) or the CTA-pair (1) kernel; default: automatic')
    args = ap.parse_args()
    shapes = [tuple(args.shape)] if args.shape else SHAPES
    for shape in shapes:
        run_shape(*shape, iters=args.iters, zipf=args.zipf, only=args.case, warmup=args.warmup, pair=args.pair)


if __name__ == '__main__':
    main()
