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
    ext().ep_wait_flags(flags, 2, 5, 19)
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
