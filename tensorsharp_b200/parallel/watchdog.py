"""Host-side liveness of the ranks of one job.

Each rank bumps a counter in the job's key-value store between steps; before a step that would block in
a collective or in an in-kernel exchange, a rank can ask whether every peer has reported recently and
get a typed error instead of a hang.  A departing rank says so explicitly (``leave``) so the others
learn of it before their next launch.  Nothing here touches a GPU: failures are detected and injected
on the host (the reference has no multi-process path and therefore no counterpart).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, Optional, Set

from .errors import RankFailureError


class Heartbeat:
    def __init__(self, store, rank: int, size: int, prefix: str = "tsb/hb", clock: Callable[[], float] = time.monotonic):
        self.store, self.rank, self.size, self.prefix, self.clock = store, rank, size, prefix, clock
        self._seen: Dict[int, tuple] = {}            # rank -> (last counter value, local time it changed)
        self._count = 0
        self.beat()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def leave(self) -> None:
        """Announce an orderly departure: peers see it at their next check."""
        self.store.set(self._key(self.rank), "left")

    def _read(self, r: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            v = self.store.get(self._key(r))
            return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
        except Exception:
            return None

    def stale_ranks(self, timeout_s: float) -> Set[int]:
        now = self.clock()
        stale: Set[int] = set()
        for r in range(self.size):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == "left":
                stale.add(r)
                continue
            # a key that is still absent (the peer has not registered yet) is one more unchanged value: the peer
            # is stale only once nothing has changed for ``timeout_s``, so start-up skew within the timeout is fine
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > timeout_s:
                stale.add(r)
        return stale

    def check(self, timeout_s: float) -> None:
        stale = self.stale_ranks(timeout_s)
        if stale:
            raise RankFailureError(stale)


class Watchdog:
    """Background thread: beats for this rank and calls ``on_failure(stale)`` once when a peer goes quiet."""

    def __init__(self, hb: Heartbeat, timeout_s: float, interval_s: float = 0.2, on_failure: Optional[Callable] = None):
        self.hb, self.timeout_s, self.interval_s, self.on_failure = hb, timeout_s, interval_s, on_failure
        self.failed: Set[int] = set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="tsb-watchdog", daemon=True)

    def start(self) -> "Watchdog":
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            self.hb.beat()
            stale = self.hb.stale_ranks(self.timeout_s)
            if stale and not self.failed:
                self.failed = set(stale)
                if self.on_failure is not None:
                    self.on_failure(self.failed)

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2)
