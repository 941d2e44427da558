"""Bandwidth-bound kernels around the MoE layers: LayerNorm (with the fused residual add),
cross-entropy, bias-gradient column sum and the fused Adam step.

Reports milliseconds and the achieved fraction of the measured copy bandwidth
(MEASURED_PEAKS.json at the repository root, 6650 GB/s if absent).

    python -m megablocks_b200.benchmarks.fused_ops_benchmark [--rows 32768] [--hidden 768] [--case NAME]
"""

import argparse

import torch

from megablocks_b200._ext import ext
from megablocks_b200.benchmarks.permute_benchmark import measured_hbm_gbs
from megablocks_b200.benchmark_util import benchmark_function
from megablocks_b200.ops import fused
from megablocks_b200.optim import FusedAdam


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--rows', type=int, default=32768)
    ap.add_argument('--hidden', type=int, default=768)
    ap.add_argument('--vocab', type=int, default=51200)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--case', type=str, default=None, help='run only the cases whose name starts with this')
    args = ap.parse_args()
    dev = torch.device('cuda')
    dt = torch.bfloat16
    peak, kind = measured_hbm_gbs()
    rows, h = args.rows, args.hidden
    act = rows * h * 2   # bytes of one activation tensor

    ln = fused.LayerNorm(h).to(device=dev, dtype=dt)
    a = torch.randn(rows, h, device=dev, dtype=dt, requires_grad=True)
    b = torch.randn(rows, h, device=dev, dtype=dt, requires_grad=True)
    ds, dy = torch.randn_like(a), torch.randn_like(a)
    lin_dy = torch.randn(rows, 3 * h, device=dev, dtype=dt)

    def ln_fwd():
        with torch.no_grad():
            ln(a)

    def add_ln_fwd():
        with torch.no_grad():
            ln.add_forward(a, b)

    def add_ln_fwd_bwd():
        s, y = ln.add_forward(a, b)
        torch.autograd.backward([s, y], [ds, dy])

    cases = {
        'layernorm forward': (ln_fwd, 2 * act),
        'add + layernorm forward': (add_ln_fwd, 4 * act),
        'add + layernorm forward + backward': (add_ln_fwd_bwd, 4 * act + 4 * act),
        'bias gradient (column sum) of [rows, 3h]': (lambda: ext().column_sum(lin_dy), 3 * act),
    }

    small_rows = min(rows, 8192)   # 8192 x 51200 bf16 logits = 0.84 GB
    logits = torch.randn(small_rows, args.vocab, device=dev, dtype=dt)
    targets = torch.randint(0, args.vocab, (small_rows,), device=dev)

    def ce_fwd_bwd():
        x = logits.detach().clone().requires_grad_(True)
        fused.cross_entropy(x, targets).backward()

    cases['cross-entropy forward + backward (+ one copy)'] = (ce_fwd_bwd, 5 * logits.numel() * 2)

    params = [torch.nn.Parameter(torch.randn(64, 3072, h, device=dev, dtype=dt)) for _ in range(2)]
    for p in params:
        p.grad = torch.randn_like(p) * 0.01
    opt = FusedAdam(params, lr=1e-3)
    n = sum(p.numel() for p in params)
    cases['fused Adam step'] = (opt.step, 28 * n)

    for name, (fn, nbytes) in cases.items():
        if args.case is not None and not name.startswith(args.case):
            continue
        mean, std = benchmark_function(fn, iterations=args.iters, warmup=args.warmup, flush_l2=True)
        gbs = nbytes / mean / 1e6
        print(f'  {name:46s} {mean * 1e3:9.1f} us +- {std * 1e3:6.1f}  {gbs:7.0f} GB/s  '
              f'{gbs / peak:5.2f} of {kind} copy bandwidth')


if __name__ == '__main__':
    main()
