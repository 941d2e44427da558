"""Failure detection without faulting a GPU.

Host side (CPU, gloo): a rank that leaves between steps is noticed by the heartbeat,
and a collective the missing rank never joins ends with an error inside the process
group timeout instead of hanging.  Device side (one GPU): a wait on a flag that
nobody sets runs into its bound, records a status code that the host turns into an
exception, and leaves the CUDA context usable.
"""

import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _heartbeat_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from megablocks_b200.utils.health import Heartbeat, PeerLost
    hb = Heartbeat(timeout_s=1.5, max_lag=1)
    result = 'ok'
    try:
        for step in range(6):
            if rank == 1 and step == 3:
                # Leaves between steps with nothing in flight (no collective is pending).
                break
            hb.beat()
            hb.check()
            time.sleep(0.05)
    except PeerLost as exc:
        result = f'lost:{exc.ranks}'
    with open(os.path.join(out_dir, f'hb{rank}.txt'), 'w') as f:
        f.write(result)
    # No barrier on the way out: rank 1 is "gone".


def test_heartbeat_reports_a_rank_that_left(tmp_path):
    mp.spawn(_heartbeat_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / 'hb0.txt').read() == 'lost:[1]'
    assert open(tmp_path / 'hb1.txt').read() == 'ok'


def _collective_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    x = torch.ones(4)
    dist.all_reduce(x)           # step 0: everybody is here
    outcome = 'ok'
    if rank == 1:
        outcome = 'left'         # never joins the second collective
    else:
        t0 = time.monotonic()
        try:
            dist.all_reduce(x)
            outcome = 'no-error'
        except Exception:
            outcome = f'error-after-{time.monotonic() - t0:.0f}s'
    with open(os.path.join(out_dir, f'c{rank}.txt'), 'w') as f:
        f.write(outcome)
    os._exit(0)                  # skip process-group teardown, which would wait for the missing peer


def test_collective_with_a_missing_rank_errors_instead_of_hanging(tmp_path):
    mp.spawn(_collective_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / 'c0.txt').read().startswith('error-after-')
    assert open(tmp_path / 'c1.txt').read() == 'left'


@pytest.mark.gpu
def test_device_wait_runs_into_its_bound_and_reports():
    from megablocks_b200._ext import ext
    from megablocks_b200.ops import gg as G
    from megablocks_b200.utils import status
    dev = torch.device('cuda', 0)
    status.read(clear=True)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)      # nobody will ever set these
    t0 = time.monotonic()
    ext().ep_wait_flags(flags, 2, 5, 19, None)
    torch.cuda.synchronize()
    assert 1.0 < time.monotonic() - t0 < 20.0
    with pytest.raises(status.DeviceWaitTimeout, match='never returned'):
        status.check()
    assert status.read() == 0                                   # cleared by check()

    # The same for the GEMM's producer warp waiting for rows that never arrive.
    a = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    w = torch.randn(2, 128, 128, device=dev, dtype=torch.bfloat16)
    bins = torch.tensor([128, 256], dtype=torch.int32, device=dev)
    G.grouped_gemm(a, w, bins, trans_b=True, wait=(flags, 2, 2, 1))
    torch.cuda.synchronize()
    with pytest.raises(status.DeviceWaitTimeout, match='never arrived'):
        status.check()
    # The context is intact: a normal launch still works and is correct.
    out, _, _ = G.grouped_gemm(a, w, bins, trans_b=True)
    ref = torch.cat([a[:128].float() @ w[0].float().t(), a[128:].float() @ w[1].float().t()])
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-1)
    status.check()


@pytest.mark.gpu
def test_expert_parallel_exchange_fails_closed():
    """A count exchange whose peer never answers must end with a status code and make everything that
    follows on the stream inert: no store into any peer buffer, context still usable.

    One process stands in for rank 0 of a two-rank group: the "peer" is a second buffer on the same
    GPU that nobody drives, so its count flag is never set (a bounded wait that expires).
    """
    from megablocks_b200._ext import ext
    from megablocks_b200.ops import gg as G
    from megablocks_b200.utils import status
    dev = torch.device('cuda', 0)
    status.read(clear=True)
    world, experts, epr, hidden, copies = 2, 4, 2, 128, 256
    heap_bytes = 1 << 20
    heaps = [torch.zeros(heap_bytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    peer_base = torch.tensor([h.data_ptr() for h in heaps], dtype=torch.int64, device=dev)
    off_counts, off_count_flags, off_flags, off_recv, off_ret = 0, 4096, 8192, 16384, 16384 + 512 * hidden * 2
    layout = (peer_base, world, 0, experts, epr, 512, off_counts, off_count_flags)
    tpe = torch.tensor([64, 64, 64, 64], dtype=torch.int32, device=dev)
    counts = torch.full((world * experts,), 12345, dtype=torch.int32, device=dev)     # garbage on purpose
    kept = torch.full((world * experts,), 12345, dtype=torch.int32, device=dev)
    recv_bins = torch.full((epr,), 999999, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * experts + 2 * world, dtype=torch.int32, device=dev)
    t0 = time.monotonic()
    ext().ep_exchange_counts(tpe, *layout, 1, 0, counts, kept, recv_bins, scratch, None)
    torch.cuda.synchronize()
    assert 1.0 < time.monotonic() - t0 < 20.0
    assert status.read(clear=False) == 16                       # the peer never published its counts
    assert not counts.any() and not kept.any() and not recv_bins.any()   # outputs are zeros, not garbage

    # With the failure on record the push, the waiting GEMM and the return kernel do nothing.
    x = torch.randn(copies, hidden, device=dev, dtype=torch.bfloat16)
    indices = torch.arange(copies, dtype=torch.int32, device=dev)
    bins = torch.tensor([64, 128, 192, 256], dtype=torch.int32, device=dev)
    done = torch.zeros(experts, dtype=torch.int32, device=dev)
    before = [h.clone() for h in heaps]
    ext().ep_push_rows(x, indices, None, bins, kept, *layout, peer_base, off_recv, off_flags, -1, 1, 1, done, None,
                       None)
    ext().ep_return_rows(x, kept, counts, *layout, peer_base, off_ret, off_flags, 1, copies, done, None)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    w = torch.randn(epr, 128, hidden, device=dev, dtype=torch.bfloat16)
    out = torch.full((copies, 128), 7.0, device=dev, dtype=torch.bfloat16)
    t0 = time.monotonic()
    G.grouped_gemm(x, w, recv_bins, trans_b=True, wait=(flags, 2, 2, 1), c=out, zero_tail=False)
    torch.cuda.synchronize()
    assert time.monotonic() - t0 < 1.0                          # did not even start waiting
    assert torch.all(out == 7.0)                                # wrote nothing
    for h, b in zip(heaps, before):
        assert torch.equal(h, b)                                # no store reached either heap
    with pytest.raises(status.DeviceWaitTimeout, match='never published'):
        status.check()
    # The context is intact and, with the status cleared, the kernels work again.
    ref = x[:64].float() @ w[0].float().t()
    got, _, _ = G.grouped_gemm(x, w, torch.tensor([64, 128], dtype=torch.int32, device=dev), trans_b=True)
    torch.testing.assert_close(got[:64].float(), ref, rtol=2e-2, atol=2e-1)
    status.check()
