"""Device-side error reporting.

Kernels that wait on a barrier, a flag or a peer bound every wait; a wait that
runs out records a code in a per-device status word instead of trapping or
spinning forever.  :func:`check` reads that word (one device synchronisation)
and raises if a kernel gave up.
"""

import torch

from megablocks_b200._ext import ext

_MESSAGES = {
    1: 'grouped GEMM: TMA producer timed out waiting for a free shared-memory stage',
    2: 'grouped GEMM: MMA warp timed out waiting for a TMA tile',
    3: 'grouped GEMM: MMA warp timed out waiting for a free accumulator',
    4: 'grouped GEMM: epilogue timed out waiting for an accumulator',
    16: 'expert-parallel count exchange: a peer never published its counts',
    17: 'expert-parallel receive buffer overflow: more rows were routed to this rank than the buffer holds',
    18: 'grouped GEMM: rows of an expert never arrived from a peer (dispatch flag not released)',
    19: 'expert-parallel combine: a peer never returned its rows',
    20: 'expert-parallel dispatch: a peer never released its receive buffer',
    32: 'data-parallel gradient reduction: a peer never announced its bucket',
    33: 'data-parallel gradient reduction: a peer never finished reading or writing a bucket',
}


class DeviceWaitTimeout(RuntimeError):
    """A kernel abandoned a bounded wait; its outputs are not valid."""


def read(clear: bool = True) -> int:
    """Status word of the current CUDA device (0 = no error)."""
    if not torch.cuda.is_available():
        return 0
    return int(ext().read_status(clear))


def check() -> None:
    code = read(clear=True)
    if code:
        raise DeviceWaitTimeout(_MESSAGES.get(code, f'device wait timed out (code {code})'))
