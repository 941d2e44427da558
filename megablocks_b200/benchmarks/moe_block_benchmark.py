"""Fused MoE block benchmark under expert parallelism, with roofline accounting.

One dMoE layer alone, forward + backward, each rank holding ``--tokens`` tokens of
width ``--hidden`` (bf16, N(0,1)); router logits get a per-expert Zipf(s) bias so the
load is skewed.  Defaults are the block of a Mixtral-sized model: 16384 tokens x 4096,
64 experts, top-2, SwiGLU ffn 14336.  Two routes are timed with CUDA events (max over
ranks): the peer-memory route (remote stores + flags fused with the grouped GEMMs) and
the library route (NCCL all-to-all, the reference's algorithm).

The roofline of the block is the slower of (expert FLOPs / measured bf16 peak) and
(bytes that must cross NVLink / 770 GB/s measured per direction per GPU); the report
gives achieved / roofline for both routes, and the exchange's share of the step.

``--impl reference`` times the unmodified reference library instead (``baseline/_ref`` through
its public ``Arguments`` / ``dMoE`` API: permute + NCCL all_to_all + grouped_gemm), on the same
tokens, router bias and group, so the two reports can be divided.  Both report the exposed
exchange time: device time of the communication-only pieces on the compute stream.

Launch with one process per GPU::

    python -m torch.distributed.run --nproc-per-node 8 -m megablocks_b200.benchmarks.moe_block_benchmark
"""

import argparse
import json
import os
from functools import partial

import torch
import torch.distributed as dist
import torch.nn.functional as F

import megablocks_b200 as mb
from megablocks_b200.benchmarks.matmul_benchmark import measured_peak_tflops
from megablocks_b200.utils import status
from megablocks_b200.utils.metrics import comm_timer

NVLINK_GBS_MEASURED = 770.0


def measured_sustained_tflops():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get('bf16_tflops_sustained', 1400.0))
    return 1400.0


def build_layer(args, fused, device, group):
    torch.manual_seed(0)
    margs = mb.Arguments(
        hidden_size=args.hidden, ffn_hidden_size=args.ffn, moe_num_experts=args.experts, moe_top_k=args.top_k,
        mlp_type='glu' if args.glu else 'mlp', mlp_impl='grouped', memory_optimized_mlp=True,
        activation_fn=F.silu if args.glu else partial(F.gelu, approximate='tanh'), bias=False, moe_loss_weight=0.0,
        fp16=False, bf16=True, device=device, moe_expert_model_parallelism=group is not None,
        expert_parallel_group=group, ep_fused_comm=fused,
        init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.02))
    layer = mb.dMoE(margs)
    with torch.no_grad():   # Zipf-skewed routing: a fixed per-expert bias folded into the router weight
        ranks = torch.arange(1, args.experts + 1, dtype=torch.float32, device=device)
        bias = torch.log(1.0 / ranks**args.zipf)
        layer.router.layer.weight.add_((bias / args.hidden).unsqueeze(1).to(layer.router.layer.weight.dtype))
    return layer


def build_reference_layer(args, device, group):
    """The reference's own dMoE (grouped path), same shapes, same Zipf bias."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.join(root, 'baseline'))
    os.environ.setdefault('MB_REF_GMM', args.ref_gmm)
    import ref_arm
    RefArguments, ref_dmoe, _ = ref_arm.import_reference()
    timer = ref_arm.ExposedCommTimer()
    torch.manual_seed(0)
    margs = RefArguments(
        hidden_size=args.hidden, ffn_hidden_size=args.ffn, moe_num_experts=args.experts, moe_top_k=args.top_k,
        mlp_type='glu' if args.glu else 'mlp', mlp_impl='grouped', memory_optimized_mlp=True,
        activation_fn=F.silu if args.glu else partial(F.gelu, approximate='tanh'), bias=False, moe_loss_weight=0.0,
        fp16=False, bf16=True, device=device, moe_expert_model_parallelism=group is not None,
        expert_parallel_group=group, init_method=partial(torch.nn.init.normal_, mean=0.0, std=0.02))
    layer = ref_dmoe.dMoE(margs)
    with torch.no_grad():
        ranks = torch.arange(1, args.experts + 1, dtype=torch.float32, device=device)
        bias = torch.log(1.0 / ranks**args.zipf)
        layer.router.layer.weight.add_((bias / args.hidden).unsqueeze(1).to(layer.router.layer.weight.dtype))
    return layer, timer


def time_layer(layer, x, steps, warmup, world, timer=comm_timer):
    def step():
        x.grad = None
        layer.zero_grad(set_to_none=True)
        out = layer(x)
        out.backward(x_probe)
    x_probe = torch.ones_like(x)
    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / steps], dtype=torch.float64, device=x.device)
    # Exposed exchange time, measured on extra steps so that the events do not perturb the timed ones.
    timer.reset()
    timer.enabled = True
    for _ in range(steps):
        step()
    timer.enabled = False
    exposed = torch.tensor([timer.total_ms() / steps], dtype=torch.float64, device=x.device)
    timer.reset()
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(exposed, op=dist.ReduceOp.MAX)
    status.check()
    return float(ms), float(exposed)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--tokens', type=int, default=16384)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--ffn', type=int, default=14336)
    ap.add_argument('--experts', type=int, default=64)
    ap.add_argument('--top-k', dest='top_k', type=int, default=2)
    ap.add_argument('--no-glu', dest='glu', action='store_false')
    ap.add_argument('--zipf', type=float, default=1.1)
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    ap.add_argument('--ref-gmm', dest='ref_gmm', choices=['loop', 'grouped_mm'], default='loop')
    args = ap.parse_args()

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29517')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
        group = dist.group.WORLD
    torch.manual_seed(1 + rank)
    x = torch.randn(args.tokens, 1, args.hidden, device=device, dtype=torch.bfloat16).requires_grad_(True)

    results, exposed = {}, {}
    if args.impl == 'reference':
        layer, timer = build_reference_layer(args, device, group)
        results['reference'], exposed['reference'] = time_layer(layer, x, args.steps, args.warmup, world, timer)
        routes = []
    else:
        routes = [('fused', True), ('nccl', False)] if world > 1 else [('local', None)]
    for name, fused in routes:
        layer = build_layer(args, fused, device, group)
        results[name], exposed[name] = time_layer(layer, x, args.steps, args.warmup, world)
        del layer
        torch.cuda.empty_cache()

    if rank == 0:
        peak, kind = measured_peak_tflops()
        sustained = measured_sustained_tflops()
        gemms = 3 if args.glu else 2
        copies = args.tokens * args.top_k
        flops = 3 * gemms * 2.0 * copies * args.hidden * args.ffn           # forward + 2x backward, per rank
        t_compute = flops / (peak * 1e12) * 1e3
        # Forward dispatch + return and the same two transfers in backward; (W-1)/W of the rows leave the GPU.
        nvlink_bytes = 4.0 * copies * args.hidden * 2 * (world - 1) / max(world, 1)
        t_link = nvlink_bytes / (NVLINK_GBS_MEASURED * 1e9) * 1e3
        roof = max(t_compute, t_link)
        roof_sustained = max(flops / (sustained * 1e12) * 1e3, t_link)
        report = {'world': world, 'impl': args.impl, 'config': vars(args), 'ms': results, 'exposed_comm_ms': exposed,
                  'roofline_ms': {'compute': t_compute, 'nvlink': t_link, 'bound': roof,
                                  'bound_at_sustained_peak': roof_sustained,
                                  'peak': f'{peak:.0f} TFLOP/s burst / {sustained:.0f} sustained ({kind}), '
                                          f'{NVLINK_GBS_MEASURED:.0f} GB/s per direction'},
                  'fraction_of_roofline': {k: roof / v for k, v in results.items()},
                  'fraction_of_roofline_sustained': {k: roof_sustained / v for k, v in results.items()},
                  'peak_mem_gb': torch.cuda.max_memory_allocated() / 1e9}
        print(json.dumps(report))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
