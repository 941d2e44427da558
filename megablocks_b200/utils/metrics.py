"""Structured training metrics and phase ranges.

The reference's observability is a pair of module-level loss lists and a
``log_benchmark`` print (megablocks/layers/moe.py:14-29, benchmark_util.py:8-16).
This module adds what a production run needs around the same layers:

* :class:`JsonlLogger` - one JSON object per line (step, loss, tokens/s, grad
  norm, per-layer expert load statistics, dropped copies), rank 0 only unless
  asked otherwise;
* :func:`expert_load_stats` - balance statistics of a ``tokens_per_expert`` vector
  computed on the device (one small copy when logged);
* :func:`nvtx_range` - NVTX ranges around phases (route / dispatch / experts /
  combine / reduce / optimizer) that cost nothing when no profiler is attached;
* :class:`DeviceTimer` - CUDA-event timing of a code region on the current stream.
"""

import contextlib
import json
import os
import time
from typing import Dict, Optional

import torch


class JsonlLogger:

    def __init__(self, path: Optional[str], rank: int = 0, all_ranks: bool = False):
        self.enabled = path is not None and (all_ranks or rank == 0)
        self.rank = rank
        self._file = None
        if self.enabled:
            os.makedirs(os.path.dirname(os.path.abspath(path)) or '.', exist_ok=True)
            self._file = open(path if not all_ranks else f'{path}.rank{rank}', 'a', buffering=1)

    def log(self, **fields) -> None:
        if not self.enabled:
            return
        record = {'time': time.time(), 'rank': self.rank}
        for key, value in fields.items():
            if isinstance(value, torch.Tensor):
                value = value.detach().float().cpu().tolist() if value.numel() > 1 else float(value)
            record[key] = value
        self._file.write(json.dumps(record) + '\n')

    def close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None


def expert_load_stats(tokens_per_expert: torch.Tensor) -> Dict[str, float]:
    """max / mean load ratio, fraction of idle experts and the coefficient of variation."""
    counts = tokens_per_expert.detach().float()
    mean = counts.mean().clamp_min(1e-9)
    stats = torch.stack([counts.max() / mean, (counts == 0).float().mean(), counts.std(unbiased=False) / mean])
    imbalance, idle, cv = stats.cpu().tolist()
    return {'max_over_mean': imbalance, 'idle_fraction': idle, 'cv': cv}


def dropped_copies(tokens_per_expert: torch.Tensor, capacity: int) -> torch.Tensor:
    """Routed copies a token-dropping MoE discards at the given per-expert capacity (device scalar)."""
    return (tokens_per_expert - capacity).clamp_min(0).sum()


@contextlib.contextmanager
def nvtx_range(name: str):
    pushed = False
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        pushed = True
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """``with DeviceTimer() as t: ...`` then ``t.ms`` (synchronises when read)."""

    def __enter__(self):
        self._start = torch.cuda.Event(enable_timing=True)
        self._end = torch.cuda.Event(enable_timing=True)
        self._start.record()
        return self

    def __exit__(self, *exc):
        self._end.record()
        return False

    @property
    def ms(self) -> float:
        self._end.synchronize()
        return self._start.elapsed_time(self._end)


class CommTimer:
    """Device time spent in communication-only work on the compute stream.

    The expert-parallel exchange brackets the kernels (or collectives) that move tokens but compute
    nothing - count exchange, dispatch push, waits for returned rows, all-to-alls of the library route
    - with :meth:`region`.  While :attr:`enabled` is false that costs nothing; while it is true every
    region records two CUDA events on the current stream, and :meth:`total_ms` adds up their
    distances after one synchronisation.  Because the regions sit on the stream the expert GEMMs
    wait behind, the sum is the exchange time that is exposed, i.e. not hidden under compute.
    """

    def __init__(self):
        self.enabled = False
        self._pairs = []

    @contextlib.contextmanager
    def region(self):
        if not self.enabled or not torch.cuda.is_available():
            yield
            return
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            end.record()
            self._pairs.append((start, end))

    def reset(self) -> None:
        self._pairs = []

    def total_ms(self) -> float:
        if not self._pairs:
            return 0.0
        torch.cuda.synchronize()
        return float(sum(s.elapsed_time(e) for s, e in self._pairs))


comm_timer = CommTimer()
