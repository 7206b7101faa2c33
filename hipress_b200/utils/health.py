"""Failure detection on the host: heartbeats through the job's key-value store, a
stall inspector, and an abort path that never involves the GPU.

Every rank bumps ``hb/<rank>`` from a daemon thread; ``HealthMonitor.check()``
(called between steps, before the next launch) raises ``PeerFailure`` when a
peer's counter stopped moving for ``timeout_s``.  A rank that wants to leave does
so between steps with nothing in flight and announces it with ``leave()``.  Device
side waits are bounded separately (csrc/cuda/sync.cuh) and surface as
``HipressTimeoutError``; recovery is: abort the step, re-rendezvous on the CPU,
restore the last checkpoint.  Upstream Horovod's stall inspector / elastic mode is
the nearest analogue; the reference tree has neither.
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks, reason):
        super().__init__(f"ranks {sorted(ranks)} {reason}")
        self.ranks = sorted(ranks)


class HealthMonitor:
    def __init__(self, store, rank: int, world: int, *, interval_s: float = 0.2,
                 timeout_s: float = 3.0, prefix: str = "hipress"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._seen = {r: (-1, time.time()) for r in range(world)}
        self._paused = False
        self.store.add(self._key(rank), 1)
        self._t = threading.Thread(target=self._beat, daemon=True)
        self._t.start()

    def _key(self, r):
        return f"{self.prefix}/hb/{r}"

    def _beat(self):
        while not self._stop.wait(self.interval_s):
            if not self._paused:
                try:
                    self.store.add(self._key(self.rank), 1)
                except Exception:
                    return

    def pause(self, on=True):
        """Test hook: stop beating without exiting (a hung host thread)."""
        self._paused = on

    def leave(self):
        """Announce an orderly exit (between steps, nothing in flight)."""
        self.store.set(f"{self.prefix}/left/{self.rank}", b"1")
        self.close()

    def check(self):
        """Raise PeerFailure if a peer left or stopped beating."""
        now = time.time()
        dead, left = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if self.store.check([f"{self.prefix}/left/{r}"]):
                    left.append(r)
                    continue
            except Exception:
                pass
            try:
                v = int(self.store.add(self._key(r), 0))
            except Exception:
                dead.append(r)
                continue
            last_v, last_t = self._seen[r]
            if v != last_v:
                self._seen[r] = (v, now)
            elif now - last_t > self.timeout_s:
                dead.append(r)
        if left:
            raise PeerFailure(left, "left the job")
        if dead:
            raise PeerFailure(dead, f"sent no heartbeat for {self.timeout_s:.1f} s")

    def close(self):
        self._stop.set()


def default_store():
    """The store of the default process group (TCPStore created by init_process_group)."""
    from torch.distributed.distributed_c10d import _get_default_store
    return _get_default_store() if dist.is_initialized() else None
