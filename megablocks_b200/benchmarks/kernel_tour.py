"""One launch of every kernel of the library on a mid-sized input, with CUDA-event timings.

Meant to be run twice: plain, for the timings it prints (L2 flushed before every launch, median of
``--iters`` launches, achieved GB/s or TFLOP/s against the measured peaks), and under Nsight
Compute on one GPU for per-kernel counters, e.g.::

    python -m megablocks_b200.benchmarks.kernel_tour --iters 5
    ncu --section SpeedOfLight --section MemoryWorkloadAnalysis --clock-control none \\
        -k regex:'mb::' -o tour python -m megablocks_b200.benchmarks.kernel_tour --iters 1 --no-timing

Inputs are larger than the 126 MB L2 wherever the kernel is bandwidth-bound and stay below 3 GB on
the device in total.
"""

import argparse
import json
import os
import statistics

import torch
import torch.nn.functional as F

from megablocks_b200 import ops
from megablocks_b200._ext import ext
from megablocks_b200.ops import fused, gg as G, sparse
from megablocks_b200.optim import FusedAdam, clip_coefficient


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d['hbm_gbs']), float(d['bf16_tflops']), 'measured'
    return 6650.0, 1590.0, 'fallback'


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--iters', type=int, default=5)
    ap.add_argument('--no-timing', action='store_true', help='launch everything once per iteration without events')
    ap.add_argument('--only', type=str, default=None, help='run only the cases whose name contains this')
    args = ap.parse_args()
    dev = torch.device('cuda')
    torch.manual_seed(0)
    hbm, tflops, kind = _peaks()
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    cases = []     # (name, fn, bytes moved or None, flops or None)

    def add(name, fn, nbytes=None, flops=None):
        if args.only is None or args.only in name:
            cases.append((name, fn, nbytes, flops))

    # ---- routing metadata -----------------------------------------------------------------
    T, E, H = 131072, 64, 768
    top = torch.randint(0, E, (T,), device=dev, dtype=torch.int32)
    add('route_plan (sort + counts + bins, 3 kernels)', lambda: ops.route_plan(top, E, 128), nbytes=T * 4 * 4)
    indices, bin_ids, bins, padded_bins, tpe = ops.route_plan(top, E, 128)
    add('histogram', lambda: ops.histogram(top, E), nbytes=T * 4)
    add('inclusive_cumsum [4096, 64]', lambda: ops.inclusive_cumsum(torch.ones(4096, 64, device=dev, dtype=torch.int32), 1))
    x = torch.randn(T, H, device=dev, dtype=bf)
    w = torch.rand(T, device=dev, dtype=bf)
    add('gather (token order -> expert order)', lambda: ops.gather(x, indices, bin_ids, bins, 1), nbytes=2 * T * H * 2)
    xg = ops.gather(x, indices, bin_ids, bins, 1)
    add('scatter (expert order -> token order, weighted)', lambda: ops.scatter(xg, indices, bin_ids, w, bins, 1),
        nbytes=2 * T * H * 2)
    add('padded_gather', lambda: ops.padded_gather(x, indices, bin_ids, bins, padded_bins, 1, num_rows=T + E * 128),
        nbytes=2 * T * H * 2)
    logits = torch.randn(T, E, device=dev, dtype=bf)
    add('router softmax + top-k forward', lambda: ext().router_topk_forward(logits, 2, 0.0), nbytes=2 * T * E * 2)

    # ---- row-wise model kernels -----------------------------------------------------------
    ln = fused.LayerNorm(H).to(device=dev, dtype=bf)
    rn = fused.RMSNorm(H).to(device=dev, dtype=bf)
    res = torch.randn(T, H, device=dev, dtype=bf)
    add('LayerNorm + residual add forward', lambda: ln.add_forward(x, res), nbytes=4 * T * H * 2)
    add('RMSNorm forward', lambda: rn(x), nbytes=2 * T * H * 2)
    xr = x.clone().requires_grad_(True)
    y = ln(xr)
    gy = torch.randn_like(y)
    add('LayerNorm backward (+ weight / bias gradients)', lambda: torch.autograd.grad(y, xr, gy, retain_graph=True),
        nbytes=3 * T * H * 2)
    V, R = 51200, 8192
    lg = torch.randn(R, V, device=dev, dtype=bf)
    tg = torch.randint(0, V, (R,), device=dev)
    add('cross-entropy forward', lambda: ext().cross_entropy_forward(lg, tg), nbytes=R * V * 2)
    loss, lse = ext().cross_entropy_forward(lg, tg)
    one = torch.ones(1, device=dev)
    add('cross-entropy backward (in place)', lambda: ext().cross_entropy_backward_(lg, tg, lse, one, 1.0 / R),
        nbytes=2 * R * V * 2)
    q = torch.randn(8, 4096, 32, 128, device=dev, dtype=bf)
    inv = 1.0 / (10000.0**(torch.arange(0, 128, 2, device=dev).float() / 128))
    ang = torch.outer(torch.arange(4096, device=dev).float(), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    add('rotary embedding', lambda: fused.rope(q, cos, sin), nbytes=2 * q.numel() * 2)
    scores = [torch.rand(32768, E, device=dev, dtype=bf).requires_grad_(True) for _ in range(12)]
    counts = [torch.randint(0, 1024, (E,), device=dev, dtype=torch.int32) for _ in range(12)]
    add('load-balancing loss forward (12 layers)', lambda: fused.load_balancing_loss(scores, counts, 1e-6),
        nbytes=12 * 32768 * E * 2)
    lbl = fused.load_balancing_loss(scores, counts, 1e-6)
    add('load-balancing loss backward (12 layers)', lambda: torch.autograd.grad(lbl, scores, retain_graph=True),
        nbytes=12 * 32768 * E * 2)
    add('column sum (bias gradient)', lambda: ext().column_sum(x), nbytes=T * H * 2)

    # ---- optimizer ----------------------------------------------------------------------
    P = 96 << 20
    param = torch.zeros(P, device=dev, dtype=bf)
    param.grad = torch.randn(P, device=dev, dtype=bf)
    opt = FusedAdam([param], lr=1e-4)
    sq = torch.zeros(1, device=dev)
    add('gradient squared norm', lambda: opt.add_sqnorm(sq), nbytes=P * 2)
    coeff = clip_coefficient(torch.ones(1, device=dev), 1.0)
    add('fused Adam (fp32 master + moments, bf16 shadow)', lambda: opt.step(coeff[0:1]), nbytes=P * 28)

    # ---- expert GEMMs -------------------------------------------------------------------
    tok, hid, ffn, ne = 32768, 768, 3072, 64
    gb = torch.cumsum(torch.bincount(torch.randint(0, ne, (tok,)), minlength=ne), 0).int().to(dev)
    gx = torch.randn(tok, hid, device=dev, dtype=bf)
    gh = torch.randn(tok, ffn, device=dev, dtype=bf)
    gw = torch.randn(ne, ffn, hid, device=dev, dtype=bf) * 0.02
    fl = 2.0 * tok * hid * ffn
    for pair, tag in ((0, 'single CTA'), (1, 'CTA pair')):
        add(f'grouped GEMM NT, {tag}', lambda pair=pair: G.grouped_gemm(gx, gw, gb, trans_b=True, pair=pair), flops=fl)
        add(f'grouped GEMM NT + GELU, {tag}', lambda pair=pair: G.grouped_gemm(gx, gw, gb, trans_b=True, epilogue=G.EPI_ACT,
                                                                               act=G.ACT_GELU_TANH, pair=pair), flops=fl)
        add(f'grouped GEMM NN, {tag}', lambda pair=pair: G.grouped_gemm(gh, gw, gb, pair=pair), flops=fl)
        add(f'grouped GEMM TN (weight gradient), {tag}',
            lambda pair=pair: G.grouped_gemm(gh, gx, gb, trans_a=True, num_groups=ne, pair=pair), flops=fl)

    # ---- block-sparse products ------------------------------------------------------------
    M = N = 8192
    K = 1024
    topo = sparse.random_mask(M, N, 0.5, 128, dtype=torch.float32)
    topo = sparse.Matrix(topo.size(), torch.randn(topo.data.shape, dtype=bf, device=dev) * 0.1,
                         topo.row_indices.to(dev), topo.column_indices.to(dev), topo.offsets.to(dev),
                         topo.column_indices_t.to(dev), topo.offsets_t.to(dev), topo.block_offsets_t.to(dev))
    nnz = topo.data.shape[0]
    a = torch.randn(M, K, device=dev, dtype=bf) * 0.1
    b = torch.randn(K, N, device=dev, dtype=bf) * 0.1
    d = torch.randn(N, K, device=dev, dtype=bf) * 0.1
    sfl = 2.0 * nnz * 128 * 128 * K
    add('block-sparse sdd (50 % of 8192 x 8192, K = 1024)', lambda: sparse.sdd(a, b, topo), flops=sfl)
    add('block-sparse dsd', lambda: sparse.dsd(topo, d), flops=sfl)
    add('block-sparse dsd, transposed topology', lambda: sparse.dsd(topo.t(), a), flops=sfl)
    dt = d.t().contiguous()          # [K, M] times the [M, N] topology
    add('block-sparse dds', lambda: sparse.dds(dt, topo), flops=sfl)

    def timed(fn):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e)

    print(f'peaks ({kind}): {hbm:.0f} GB/s copy, {tflops:.0f} TFLOP/s bf16')
    for name, fn, nbytes, flops in cases:
        fn()                      # warm-up (also builds lazily created state)
        torch.cuda.synchronize()
        if args.no_timing:
            for _ in range(args.iters):
                fn()
            torch.cuda.synchronize()
            continue
        ms = statistics.median(timed(fn) for _ in range(args.iters))
        note = ''
        if nbytes:
            gbs = nbytes / ms / 1e6
            note = f'{gbs:8.0f} GB/s  {gbs / hbm:5.2f} of {kind} copy bandwidth'
        if flops:
            tf = flops / ms / 1e9
            note = f'{tf:8.0f} TFLOP/s {tf / tflops:5.2f} of {kind} bf16 peak'
        print(f'{name:58s} {ms:8.3f} ms  {note}')
    from megablocks_b200.utils import status
    status.check()


if __name__ == '__main__':
    main()
