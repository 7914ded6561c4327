"""Host-side failure detection: a per-rank step watchdog and a store-based heartbeat.

The reference only has the NCCL timeout (``--distributed-timeout-minutes``, ``run_unified.sh:71``): a
dead producer or a hung collective stalls every rank for an hour.  Here a rank (a) aborts itself
with a diagnostic when one step exceeds ``--step-timeout-seconds`` and (b) can publish heartbeats
into the rendezvous store so peers learn of a departed rank *on the host*, between steps, before
launching their next collective.  Nothing here touches the GPU.
"""

from __future__ import annotations

import os
import sys
import threading
import time
from typing import Callable, Dict, List, Optional


class StepWatchdog:
    """Background thread: if ``beat()`` is not called for ``timeout`` seconds, run ``on_timeout``
    (default: print a diagnostic and ``os._exit(75)`` so the launcher can restart from the last
    checkpoint)."""

    def __init__(self, timeout: float, on_timeout: Optional[Callable[[int, float], None]] = None, poll: float = 0.25):
        self.timeout, self.poll = timeout, poll
        self.on_timeout = on_timeout or self._abort
        self._last = time.monotonic()
        self._step = -1
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
        self._thread.start()

    def beat(self, step: int) -> None:
        self._last = time.monotonic()
        self._step = step

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2.0)

    def _run(self):
        while not self._stop.wait(self.poll):
            idle = time.monotonic() - self._last
            if idle > self.timeout:
                self.fired = True
                self.on_timeout(self._step, idle)
                return

    @staticmethod
    def _abort(step: int, idle: float):
        print(f"[watchdog] step {step} made no progress for {idle:.1f}s; aborting this rank", file=sys.stderr, flush=True)
        os._exit(75)


class Heartbeat:
    """Rank liveness through a ``torch.distributed`` key-value store (TCPStore / FileStore / HashStore).

    Every rank periodically writes ``hb/<rank> = <monotonic counter>``; ``dead_ranks()`` lists peers
    whose counter has not advanced within ``timeout`` seconds as seen by this rank's clock.
    """

    def __init__(self, store, rank: int, world_size: int, timeout: float = 5.0):
        self.store, self.rank, self.world_size, self.timeout = store, rank, world_size, timeout
        self._count = 0
        self._seen: Dict[int, int] = {}
        self._seen_at: Dict[int, float] = {}
        self.beat()

    def beat(self) -> None:
        self._count += 1
        self.store.set(f"hb/{self.rank}", str(self._count))

    def leave(self) -> None:
        """Announce an orderly departure (between steps, nothing in flight)."""
        self.store.set(f"hb/{self.rank}", "left")

    def dead_ranks(self) -> List[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"hb/{r}").decode()
            except Exception:
                v = None
            if v == "left":
                dead.append(r)
                continue
            c = int(v) if v is not None else -1
            if self._seen.get(r) != c:
                self._seen[r], self._seen_at[r] = c, now
            elif now - self._seen_at.get(r, now) > self.timeout:
                dead.append(r)
        return dead
