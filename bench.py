"""Headline benchmark: dMoE training throughput (tokens/s per box, max over ranks).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...             # the unmodified reference

Model and step are the reference's 125M dMoE experiment (exp/dmoe/dmoe_125m_8gpu.sh
of the reference): GPT-2 backbone with 12 layers, d_model 768, 12 heads, seq 1024,
vocab 51200, every FFN a dMoE with 64 experts, top-1, ffn 3072, tanh-GELU; bf16
compute with fp32 master weights, Adam, clip-grad 1.0; micro-batch 32 per GPU;
expert-parallel degree = number of GPUs with the non-expert parameters
data-parallel.  Tokens are uniform-random ids, weights are randomly initialised.

For N > 1 the script expects to be started once per GPU (``python -m
torch.distributed.run --nproc-per-node N bench.py --gpus N ...``) and reads
RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment.

Two numbers are measured back to back, both with CUDA events between a barrier +
device synchronisation on each side and reduced with MAX over ranks:
``value`` with inputs already on the device and no host synchronisation inside the
timed region, and ``e2e`` through ``Trainer.run_from_host`` (the training-loop call) where
every step copies its token batch from pinned host memory and every step's loss is read
back to the host (the loop waits for the loss of step k once step k + 1 is queued; all
losses are on the host before the timed region ends).  Rank 0 prints one JSON line.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = 'dMoE train tokens/s per box (max over ranks)'
MODEL = dict(layers=12, hidden=768, heads=12, seq=1024, vocab=51200, experts=64, top_k=1, ffn=3072)
MICRO_BATCH = 32
# Throughput derived from the reference's published training-time plot for this model
# on 8x A100-80GB (0.19 days for 20000 steps x 512 x 1024 tokens): 80k tokens/s per GPU.
PUBLISHED_TOKENS_PER_S_PER_GPU = 80_000.0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.gpu_index, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits', '-lms', '200', '-i',
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[4:8]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'samples': len(sm), 'reasons': sorted(reasons)}


def _dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if world != n_gpus:
        raise SystemExit(f'--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run '
                         f'--nproc-per-node {n_gpus}')
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29511')
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', local))
    return rank, world, local


def _measure(trainer, world, rank, local, steps, warmup, launch_counter, comm_timer=None):
    """Returns (device-timed ms/step, e2e ms/step, clocks, launches, h2d bytes, d2h bytes, loss, exposed comm ms)."""
    import torch
    import torch.distributed as dist

    device = torch.device('cuda', local)
    gen = torch.Generator().manual_seed(1234 + rank)
    seq, vocab = MODEL['seq'], MODEL['vocab']
    host_batches = [torch.randint(0, vocab, (MICRO_BATCH, seq + 1), generator=gen).pin_memory() for _ in range(4)]
    dev_batches = [b.to(device) for b in host_batches]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(warmup):
        b = dev_batches[i % len(dev_batches)]
        trainer.step(b[:, :-1], b[:, 1:])
    barrier()

    sampler = ClockSampler(local)
    sampler.start()
    launches0 = launch_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        b = dev_batches[i % len(dev_batches)]
        trainer.step(b[:, :-1], b[:, 1:])
    _flush(trainer)   # deferred optimizer work of the last step belongs to the timed region
    end.record()
    barrier()
    launches = launch_counter() - launches0
    device_ms = max_over_ranks(start.elapsed_time(end) / steps)
    trainer.graph_used = getattr(trainer, '_graph', None) is not None

    # End to end: host-resident batch in, loss value out, every step.
    trainer.step_from_host(host_batches[0])
    barrier()
    start2, end2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start2.record()
    # The training-loop call of the public API: every step copies its batch from pinned host memory
    # and every step's loss comes back to the host; the loop waits for the loss of step k after it
    # has queued step k + 1.  All K losses are on the host before the region ends.
    losses = trainer.run_from_host(host_batches[i % len(host_batches)] for i in range(steps))
    assert len(losses) == steps
    last = losses[-1]
    _flush(trainer)
    end2.record()
    barrier()
    clocks = sampler.stop()
    e2e_ms = max_over_ranks(start2.elapsed_time(end2) / steps)
    h2d = host_batches[0].numel() * host_batches[0].element_size()
    # Exposed exchange time (outside both timed regions): device time of the communication-only
    # pieces of the expert-parallel exchange on the compute stream, per step, max over ranks.
    exposed = None
    if comm_timer is not None and world > 1:
        # The timer brackets the exchange with events at launch time: this pass runs kernel by
        # kernel (a replayed graph has no such events).
        if getattr(trainer, '_graph', None) is not None:
            import dataclasses
            trainer.drop_graph()
            trainer.cfg = dataclasses.replace(trainer.cfg, cuda_graph=False)
        comm_timer.reset()
        comm_timer.enabled = True
        for i in range(steps):
            b = dev_batches[i % len(dev_batches)]
            trainer.step(b[:, :-1], b[:, 1:])
        _flush(trainer)
        comm_timer.enabled = False
        exposed = max_over_ranks(comm_timer.total_ms() / steps)
        comm_timer.reset()
    return device_ms, e2e_ms, clocks, launches, h2d, 4, last, exposed


def _flush(trainer):
    flush = getattr(trainer, 'flush', None)
    if flush is not None:
        flush()


def _emit(impl, n_gpus, steps, warmup, device_ms, e2e_ms, clocks, launches, h2d, d2h, loss, exposed,
          extra_config=None):
    tokens_per_step = n_gpus * MICRO_BATCH * MODEL['seq']
    value = tokens_per_step / (device_ms / 1e3)
    e2e = tokens_per_step / (e2e_ms / 1e3)
    config = {
        'model': 'dMoE-XS: GPT-2 125M backbone (12L, d768, 12 heads), every FFN a dMoE 64 experts top-1 ffn 3072 GELU',
        'global_batch': n_gpus * MICRO_BATCH, 'micro_batch_per_gpu': MICRO_BATCH, 'seq_len': MODEL['seq'],
        'vocab': MODEL['vocab'], 'parallelism': f'ep{n_gpus}' + (f'+dp{n_gpus}(non-expert)' if n_gpus > 1 else ''),
        'optimizer': 'Adam, fp32 master weights, clip-grad 1.0',
        'l2': 'no flush needed: one step touches tens of GB, far beyond the 126 MB L2',
        'vs_baseline_denominator': 'reference plot-derived 80k tokens/s per A100 GPU x n_gpus',
        'last_loss': loss,
        'exposed_comm_ms': exposed,
    }
    config.update(extra_config or {})
    line = {
        'metric': METRIC, 'value': value, 'unit': 'tokens/s', 'n_gpus': n_gpus, 'steps': steps, 'warmup': warmup,
        'ms_per_step': device_ms, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': value / (PUBLISHED_TOKENS_PER_S_PER_GPU * n_gpus), 'dtype': 'bf16',
        'data': 'synthetic uniform-random token ids, random-init weights', 'impl': impl, 'config': config,
        'clocks': clocks,
        'e2e': {'value': e2e, 'unit': 'tokens/s', 'ms_per_step': e2e_ms, 'h2d_bytes_per_step': h2d,
                'd2h_bytes_per_step': d2h},
        'gpu_launches': launches,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank, world, local = _dist_setup(args.gpus)
    from megablocks_b200._ext import ext
    from megablocks_b200.models.transformer import MoETransformer, preset
    from megablocks_b200.train import Trainer, TrainerConfig
    from megablocks_b200.utils import status

    torch.manual_seed(1234)
    group = dist.group.WORLD if world > 1 else None
    fused = {'auto': None, 'fused': True, 'nccl': False}[args.ep_comm]
    cfg = preset('dmoe-125m', device=torch.device('cuda', local), expert_parallel_group=group,
                 mlp_impl=args.mlp_impl, memory_optimized_mlp=args.memory_optimized_mlp, ep_fused_comm=fused)
    model = MoETransformer(cfg)
    # The whole step is recorded in a CUDA graph during the warm-up steps (two plain steps, then
    # the recording) and the timed steps replay it.  On several ranks the peer-memory kernels of
    # the exchange and of the gradient reduction take their sequence numbers from device counters,
    # and no library collective is left in the step.
    use_graph = args.cuda_graph == 'on' or (args.cuda_graph == 'auto' and args.warmup >= 3)
    trainer = Trainer(model, TrainerConfig(lr=6e-4, total_steps=20000, cuda_graph=use_graph, graph_warmup_steps=2),
                      dp_group=group)
    from megablocks_b200.utils.metrics import comm_timer
    out = _measure(trainer, world, rank, local, args.steps, args.warmup, ext().launch_count, comm_timer)
    status.check()
    if rank == 0:
        _emit('megablocks_b200', args.gpus, args.steps, args.warmup, *out,
              extra_config={'mlp_impl': args.mlp_impl, 'memory_optimized_mlp': args.memory_optimized_mlp,
                            'cuda_graph_step': bool(getattr(trainer, 'graph_used', False)),
                            'ep_comm': ('none' if world == 1 else
                                        'fused peer-memory kernels (remote stores + flags, no NCCL all-to-all)'
                                        if model.blocks[0].moe.experts._ep_workspaces else
                                        'nccl all_to_all')})
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    os.environ['MB_REF_GMM'] = args.ref_gmm
    try:
        import torch
        import torch.distributed as dist
        sys.path.insert(0, os.path.join(ROOT, 'baseline'))
        import ref_arm
        ref_arm.import_reference()
    except Exception as exc:  # the reference (or its CUDA extension) is not installed on this box
        if int(os.environ.get('RANK', '0')) == 0:
            print(json.dumps({'impl': 'reference', 'unavailable': f'{type(exc).__name__}: {exc}'.splitlines()[0]}),
                  flush=True)
        return
    rank, world, local = _dist_setup(args.gpus)
    torch.manual_seed(1234)
    group = dist.group.WORLD if world > 1 else None
    model = ref_arm.RefGPT(MODEL, torch.device('cuda', local), ep_group=group,
                           memory_optimized_mlp=args.memory_optimized_mlp)
    comm_timer = ref_arm.ExposedCommTimer()
    trainer = ref_arm.RefTrainer(model, lr=6e-4, min_lr=6e-5, total_steps=20000, world=world, group=group)
    out = _measure(trainer, world, rank, local, args.steps, args.warmup, lambda: 0, comm_timer)
    if rank == 0:
        _emit('reference', args.gpus, args.steps, args.warmup, *out,
              extra_config={'mlp_impl': 'grouped', 'memory_optimized_mlp': args.memory_optimized_mlp,
                            'ep_comm': 'nccl all_to_all' if world > 1 else 'none',
                            'ref_gmm': args.ref_gmm,
                            'note': 'unmodified reference library from baseline/_ref; grouped_gemm and stk '
                                    'are import shims (grouped_gemm = per-expert cuBLAS loop, or one '
                                    'torch._grouped_mm launch with --ref-gmm grouped_mm), backbone/optimizer '
                                    'plain PyTorch'})
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=8)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    ap.add_argument('--mlp-impl', dest='mlp_impl', choices=['grouped', 'sparse'], default='grouped')
    ap.add_argument('--ep-comm', dest='ep_comm', choices=['auto', 'fused', 'nccl'], default='auto',
                    help='expert-parallel exchange: peer-memory kernels (auto/fused) or NCCL all-to-all')
    ap.add_argument('--cuda-graph', dest='cuda_graph', choices=['auto', 'on', 'off'], default='auto',
                    help='replay the training step from one CUDA graph (auto: on when there are at least 3 warm-up steps)')
    ap.add_argument('--ref-gmm', dest='ref_gmm', choices=['loop', 'grouped_mm'], default='loop',
                    help="reference arm only: its grouped_gemm dependency as the package's default per-expert "
                         'cuBLAS loop, or as one torch._grouped_mm launch per GEMM (the analogue of the '
                         "package's CUTLASS build)")
    ap.add_argument('--memory-optimized-mlp', dest='memory_optimized_mlp', action='store_true',
                    help='recompute the expert activation in backward (both arms); off, as in the '
                         "reference's Arguments default and its experiment scripts")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
