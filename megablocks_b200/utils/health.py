"""Host-side failure detection for multi-rank jobs.

The fused expert-parallel kernels wait on flags that peer GPUs write.  Those waits
are bounded on the device (two seconds, then a status code), but it is cheaper to
learn on the host, *before* launching, that a peer is gone.  :class:`Heartbeat`
keeps one counter per rank in the job's key-value store (the one
``init_process_group`` created): every rank bumps its own counter once per step
and, before the next step, checks that no peer has fallen further behind than
``max_lag`` steps for longer than ``timeout_s`` seconds.  A rank that left - between
steps, with nothing in flight - is reported as :class:`PeerLost` instead of
surfacing later as a collective or flag-wait timeout.

The reference has no failure detection beyond the process-group timeout of its test
fixture (tests/fixtures/autouse.py:61-66 of the reference).
"""

import time
from typing import List, Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
    """A peer rank stopped making progress."""

    def __init__(self, ranks: List[int], step: int):
        super().__init__(f'ranks {ranks} have not reached step {step}')
        self.ranks = ranks


class Heartbeat:

    def __init__(self, store: Optional[dist.Store] = None, rank: Optional[int] = None, world: Optional[int] = None,
                 prefix: str = 'mb200/heartbeat', timeout_s: float = 30.0, max_lag: int = 1):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix, self.timeout_s, self.max_lag = prefix, timeout_s, max_lag
        self.step = 0
        self.store.set(self._key(self.rank), '0')

    def _key(self, rank: int) -> str:
        return f'{self.prefix}/{rank}'

    def beat(self) -> int:
        """Announce that this rank finished another step."""
        self.step += 1
        self.store.set(self._key(self.rank), str(self.step))
        return self.step

    def peer_steps(self) -> List[int]:
        out = []
        for r in range(self.world):
            try:
                out.append(int(self.store.get(self._key(r)).decode()))
            except Exception:
                out.append(-1)
        return out

    def check(self) -> None:
        """Raise :class:`PeerLost` if some peer stays more than ``max_lag`` steps behind for ``timeout_s``."""
        need = self.step - self.max_lag
        deadline = time.monotonic() + self.timeout_s
        while True:
            behind = [r for r, s in enumerate(self.peer_steps()) if r != self.rank and s < need]
            if not behind:
                return
            if time.monotonic() > deadline:
                raise PeerLost(behind, need)
            time.sleep(min(0.05, self.timeout_s / 20))
