"""CUDA-event timing helper (reference: megablocks/benchmark_util.py:8-35).

``benchmark_function`` warms up, then times each iteration between two CUDA
events on the current stream with a device synchronisation on both sides, and
returns ``(mean_ms, std_ms)``.  ``flush_l2=True`` overwrites a buffer larger
than the 126 MB L2 between iterations so every iteration starts cold.
"""

import numpy as np
import torch

_L2_FLUSH_BYTES = 256 << 20
_flush_buffer = None


def _flush_l2():
    global _flush_buffer
    if _flush_buffer is None:
        _flush_buffer = torch.empty(_L2_FLUSH_BYTES, dtype=torch.uint8, device='cuda')
    _flush_buffer.zero_()


def log_benchmark(name, arguments, time, std):
    print('=' * 60)
    print(f'{name} Benchmark')
    print('Benchmark Parameters:')
    for key, value in arguments.items():
        print(f'{key} = {value}')
    print('Results:')
    print('mean time = {:.3f}ms, std time = {:.3f}ms'.format(time, std))
    print('=' * 60)


def benchmark_function(fn, iterations=100, warmup=10, flush_l2=False):
    for _ in range(warmup):
        fn()
    times = []
    if not torch.cuda.is_available():       # host-only runs (smoke tests of the benchmark scripts): wall clock
        import time
        for _ in range(iterations):
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
        times = np.array(times)
        return times.mean(), times.std()
    for _ in range(iterations):
        if flush_l2:
            _flush_l2()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    times = np.array(times)
    return times.mean(), times.std()
