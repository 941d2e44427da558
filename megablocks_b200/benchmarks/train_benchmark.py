"""Training-step benchmark for any preset (the other named configurations).

``bench.py`` at the repository root measures the headline 125M dMoE; this script runs
the same measurement (CUDA events, barrier + synchronise on both sides, max over
ranks) for the other models, e.g.

* dMoE-Medium, block-sparse experts, EP = DP = 8, micro-batch 16::

    torchrun --nproc-per-node 8 -m megablocks_b200.benchmarks.train_benchmark \\
        --preset dmoe-356m --mlp-impl sparse --micro-batch 16

* Mixtral-8x7B-shaped, EP = 8, ZeRO-1, activation recompute, micro-batch 1, seq 4096::

    torchrun --nproc-per-node 8 -m megablocks_b200.benchmarks.train_benchmark \\
        --preset mixtral-8x7b --micro-batch 1 --zero1 --recompute

``--impl reference`` runs the same model, batch and optimizer recipe around the unmodified
reference library (``baseline/ref_arm.py``: its ``dMoE`` on its stock grouped path inside a
plain-PyTorch backbone), for the ratio of the two JSON lines.

``--layers`` shortens the model (per-layer cost is what the measurement is after when
the full depth does not fit the GPUs at hand); the JSON line says so.
"""

import argparse
import json
import os

import torch
import torch.distributed as dist

from megablocks_b200.models.transformer import PRESETS, preset


def _build_ours(args, cfg, group):
    from megablocks_b200._ext import ext
    from megablocks_b200.models.transformer import MoETransformer
    from megablocks_b200.train import Trainer, TrainerConfig
    from megablocks_b200.utils.metrics import comm_timer
    model = MoETransformer(cfg)
    return Trainer(model, TrainerConfig(zero1=args.zero1), dp_group=group), ext().launch_count, comm_timer


def _build_reference(args, cfg, group, device, world):
    """Same shapes around the reference's dMoE.  Nothing of this library is on that path."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.join(root, 'baseline'))
    os.environ.setdefault('MB_REF_GMM', args.ref_gmm)
    import ref_arm
    ref_arm.import_reference()
    timer = ref_arm.ExposedCommTimer()
    shape = dict(hidden=cfg.hidden_size, ffn=cfg.ffn_hidden_size, layers=cfg.num_layers, heads=cfg.num_heads,
                 seq=cfg.max_seq_len, vocab=cfg.vocab_size, experts=cfg.moe_num_experts, top_k=cfg.moe_top_k,
                 flavour=cfg.flavour, kv_heads=cfg.num_kv_heads, rope_theta=cfg.rope_theta)
    model = ref_arm.RefGPT(shape, device, ep_group=group, memory_optimized_mlp=cfg.memory_optimized_mlp,
                           recompute=args.recompute)
    return ref_arm.RefTrainer(model, world=world, group=group), (lambda: 0), timer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--preset', choices=sorted(PRESETS), default='dmoe-356m')
    ap.add_argument('--layers', type=int, default=None)
    ap.add_argument('--micro-batch', type=int, default=16)
    ap.add_argument('--seq', type=int, default=None)
    ap.add_argument('--mlp-impl', choices=['grouped', 'sparse'], default='grouped')
    ap.add_argument('--zero1', action='store_true')
    ap.add_argument('--recompute', action='store_true')
    ap.add_argument('--ep-comm', choices=['auto', 'fused', 'nccl'], default='auto')
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    ap.add_argument('--ref-gmm', dest='ref_gmm', choices=['loop', 'grouped_mm'], default='loop')
    args = ap.parse_args()

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29521')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
        group = dist.group.WORLD
    torch.manual_seed(1234)
    overrides = dict(device=device, expert_parallel_group=group, mlp_impl=args.mlp_impl,
                     activation_checkpointing=args.recompute,
                     ep_fused_comm={'auto': None, 'fused': True, 'nccl': False}[args.ep_comm])
    if args.layers:
        overrides['num_layers'] = args.layers
    if args.seq:
        overrides['max_seq_len'] = args.seq
    cfg = preset(args.preset, **overrides)
    if args.impl == 'reference':
        trainer, launch_count, timer = _build_reference(args, cfg, group, device, world)
    else:
        trainer, launch_count, timer = _build_ours(args, cfg, group)
    gen = torch.Generator().manual_seed(1 + rank)
    batches = [torch.randint(0, cfg.vocab_size, (args.micro_batch, cfg.max_seq_len + 1), generator=gen).to(device)
               for _ in range(2)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        b = batches[i % 2]
        trainer.step(b[:, :-1], b[:, 1:])
    barrier()
    launches0 = launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        b = batches[i % 2]
        loss = trainer.step(b[:, :-1], b[:, 1:])
    end.record()
    barrier()
    launches = launch_count() - launches0
    ms = torch.tensor([start.elapsed_time(end) / args.steps], dtype=torch.float64, device=device)
    exposed = torch.zeros(1, dtype=torch.float64, device=device)
    if world > 1:
        timer.reset()
        timer.enabled = True
        for i in range(args.steps):
            b = batches[i % 2]
            trainer.step(b[:, :-1], b[:, 1:])
        timer.enabled = False
        exposed[0] = timer.total_ms() / args.steps
        timer.reset()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(exposed, op=dist.ReduceOp.MAX)
    if args.impl == 'ours':
        from megablocks_b200.utils import status
        status.check()
    if rank == 0:
        tokens = world * args.micro_batch * cfg.max_seq_len
        print(json.dumps({
            'impl': args.impl, 'preset': args.preset, 'layers': cfg.num_layers, 'full_depth': args.layers is None, 'n_gpus': world,
            'micro_batch': args.micro_batch, 'seq_len': cfg.max_seq_len, 'mlp_impl': args.mlp_impl,
            'zero1': args.zero1, 'recompute': args.recompute, 'ep_comm': args.ep_comm, 'ms_per_step': float(ms),
            'tokens_per_s': tokens / float(ms) * 1e3, 'loss': float(loss),
            'peak_mem_gb': torch.cuda.max_memory_allocated() / 1e9,
            'exposed_comm_ms': float(exposed), 'gpu_launches': launches}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
