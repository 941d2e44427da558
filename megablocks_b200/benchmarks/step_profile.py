"""Where a training step goes: per-kernel device time and idle gaps of rank 0, from ``torch.profiler``.

Runs the headline 125M dMoE step (or any preset) on 1..8 GPUs, profiles ``--steps`` steps on
rank 0 after warm-up and prints (a) the kernels grouped by name with their total device time per
step, (b) the time the GPU's compute stream spent idle between kernels, (c) the time inside this
library's communication-only regions (``exposed_comm_ms``: count exchange, dispatch push, waits for
returned rows) and (d) the device time of the data-parallel reduction kernels and how much of it
ran while no other kernel did.  The step time quoted in reports comes from ``bench.py`` (no profiler
attached); this script explains its composition.

    python -m torch.distributed.run --nproc-per-node 8 -m megablocks_b200.benchmarks.step_profile
"""

import argparse
import json
import os
from collections import defaultdict

import torch
import torch.distributed as dist
from torch.profiler import ProfilerActivity, profile

from megablocks_b200.models.transformer import MoETransformer, PRESETS, preset
from megablocks_b200.train import Trainer, TrainerConfig
from megablocks_b200.utils.metrics import comm_timer


def _short(name: str) -> str:
    name = name.replace('void ', '').replace('(anonymous namespace)::', '')
    for cut in ('(', '<'):
        if cut == '<' and ('grouped_gemm' in name or 'adam' in name):
            continue
        i = name.find(cut)
        if i > 0:
            name = name[:i]
    return name[:80]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--preset', choices=sorted(PRESETS), default='dmoe-125m')
    ap.add_argument('--micro-batch', type=int, default=32)
    ap.add_argument('--steps', type=int, default=2)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--dp-comm', choices=['auto', 'peer', 'nccl'], default='auto')
    ap.add_argument('--ep-comm', choices=['auto', 'fused', 'nccl'], default='auto')
    ap.add_argument('--gap-rows', dest='gap_rows', type=int, default=25)
    ap.add_argument('--rows', type=int, default=40)
    args = ap.parse_args()
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    group = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29531')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
        group = dist.group.WORLD
    torch.manual_seed(1234)
    cfg = preset(args.preset, device=dev, expert_parallel_group=group, memory_optimized_mlp=False,
                 ep_fused_comm={'auto': None, 'fused': True, 'nccl': False}[args.ep_comm])
    trainer = Trainer(MoETransformer(cfg), TrainerConfig(dp_backend=args.dp_comm), dp_group=group)
    gen = torch.Generator().manual_seed(1 + rank)
    batch = torch.randint(0, cfg.vocab_size, (args.micro_batch, cfg.max_seq_len + 1), generator=gen).to(dev)

    def step():
        trainer.step(batch[:, :-1], batch[:, 1:])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    comm_timer.reset()
    comm_timer.enabled = True
    for _ in range(args.steps):
        step()
    comm_timer.enabled = False
    exposed = comm_timer.total_ms() / args.steps
    comm_timer.reset()
    if world > 1:
        dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    end.record()
    torch.cuda.synchronize()
    plain_ms = start.elapsed_time(end) / args.steps
    if world > 1:
        dist.barrier()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if rank == 0:
        kernels = []
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA and ev.time_range is not None:
                kernels.append((ev.time_range.start, ev.time_range.end, ev.name))
        kernels.sort()
        by_name = defaultdict(lambda: [0.0, 0])
        for s, e, n in kernels:
            by_name[_short(n)][0] += (e - s) / 1e3
            by_name[_short(n)][1] += 1
        # Union of all kernel intervals (any stream) = time the GPU was busy; the rest of the span is idle.
        busy, cur_s, cur_e = 0.0, None, None
        comm_names = ('dp_allreduce', 'ncclDevKernel', 'nccl')
        comm_intervals = [(s, e) for s, e, n in kernels if any(c in n for c in comm_names)]
        other = [(s, e) for s, e, n in kernels if not any(c in n for c in comm_names)]
        gaps = defaultdict(lambda: [0.0, 0])     # (kernel before, kernel after) -> [idle us, count]
        last_name = None
        for s, e, n in kernels:
            if cur_e is None or s > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                    key = (_short(last_name)[:44], _short(n)[:44])
                    gaps[key][0] += s - cur_e
                    gaps[key][1] += 1
                cur_s, cur_e, last_name = s, e, n
            else:
                if e > cur_e:
                    cur_e, last_name = e, n
        if cur_e is not None:
            busy += cur_e - cur_s
        span = (kernels[-1][1] - kernels[0][0]) if kernels else 0.0
        # Data-parallel reduction time that no compute kernel overlapped.
        other.sort()
        merged = []
        for s, e in other:
            if merged and s <= merged[-1][1]:
                merged[-1][1] = max(merged[-1][1], e)
            else:
                merged.append([s, e])
        alone = 0.0
        for s, e in comm_intervals:
            covered = 0.0
            for ms_, me_ in merged:
                if me_ <= s:
                    continue
                if ms_ >= e:
                    break
                covered += min(e, me_) - max(s, ms_)
            alone += (e - s) - covered
        steps = args.steps
        print(json.dumps({'world': world, 'preset': args.preset, 'step_ms_without_profiler': plain_ms,
                          'profiled_span_ms_per_step': span / 1e3 / steps, 'gpu_busy_ms_per_step': busy / 1e3 / steps,
                          'idle_ms_per_step': (span - busy) / 1e3 / steps, 'exposed_ep_comm_ms_per_step': exposed,
                          'dp_reduce_kernel_ms_per_step': sum(e - s for s, e in comm_intervals) / 1e3 / steps,
                          'dp_reduce_not_overlapped_ms_per_step': alone / 1e3 / steps,
                          'kernel_launches_per_step': len(kernels) / steps}))
        print(f'{"kernel":82s} {"ms/step":>9s} {"share":>7s} {"launches/step":>14s}')
        total = sum(v[0] for v in by_name.values())
        for name, (ms, n) in sorted(by_name.items(), key=lambda kv: -kv[1][0])[:args.rows]:
            print(f'{name:82s} {ms / steps:9.3f} {ms / total:7.1%} {n / steps:14.1f}')
        # Where the GPU sat idle: gaps between the end of one kernel and the start of the next
        # (over all streams), summed per pair of neighbours.
        print(f'\n{"idle after kernel":46s} {"before kernel":46s} {"ms/step":>8s} {"gaps/step":>10s}')
        for (a, b), (us, n) in sorted(gaps.items(), key=lambda kv: -kv[1][0])[:args.gap_rows]:
            print(f'{a:46s} {b:46s} {us / 1e3 / steps:8.3f} {n / steps:10.1f}')
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
