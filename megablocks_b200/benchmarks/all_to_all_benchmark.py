"""Token exchange benchmark: NCCL all-to-all against the peer-memory push kernels.

Sizes follow the reference benchmark (megablocks/ops/all_to_all_benchmark.py:10-29):
``sl`` rows of 1024 half-precision values per rank, split evenly over the ranks.  For
every size the NCCL ``all_to_all_single`` and this library's ``ep_push_rows`` (remote
16-byte stores into the peers' buffers + release flags, followed by the flag wait)
are timed with CUDA events, max over ranks, and reported as per-GPU outgoing GB/s
against the measured 770 GB/s per direction.

    python -m torch.distributed.run --nproc-per-node 8 -m megablocks_b200.benchmarks.all_to_all_benchmark
"""

import json
import os

import torch
import torch.distributed as dist

from megablocks_b200 import ops
from megablocks_b200._ext import ext
from megablocks_b200.parallel.ep import EpWorkspace

SIZES = [2**k for k in range(10, 21)]
HIDDEN = 1024


def _time(fn, world, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / iters], dtype=torch.float64, device='cuda')
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main():
    world = int(os.environ['WORLD_SIZE'])
    rank = int(os.environ['RANK'])
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29519')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    group = dist.group.WORLD
    rows_out = []
    for sl in SIZES:
        x = torch.randn(sl, HIDDEN, device=device, dtype=torch.bfloat16)
        out = torch.empty_like(x)
        nccl_ms = _time(lambda: dist.all_to_all_single(out, x), world)
        # Same traffic through the push kernel: `world` experts, one per rank, rows dealt round-robin.
        top = (torch.arange(sl, device=device, dtype=torch.int32) % world).contiguous()
        indices, bin_ids, bins, _, tpe = ops.route_plan(top, world)
        ws = EpWorkspace(group, world, sl, HIDDEN, torch.bfloat16, device)

        def push():
            seq = ws.next_seq()
            counts, recv_bins, done = ws.exchange_counts(tpe, seq)
            ws.push(x, indices, None, bins, counts, 0, seq, 1, done[0])
            flags, count, stride, _ = ws.arrival(0, seq)
            ext().ep_wait_flags(flags, count * stride, seq, 19, None)
            ws.release_receive_buffer(seq)

        push_ms = _time(push, world)
        sent = sl * HIDDEN * 2 * (world - 1) / world
        rows_out.append({'rows': sl, 'nccl_ms': nccl_ms, 'push_ms': push_ms, 'nccl_gbs': sent / nccl_ms / 1e6,
                         'push_gbs': sent / push_ms / 1e6, 'push_fraction_of_770': sent / push_ms / 1e6 / 770.0})
        del ws
    if rank == 0:
        for r in rows_out:
            print(json.dumps(r))
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
