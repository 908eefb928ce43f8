"""Rank liveness over the rendezvous store.

Every rank bumps a per-rank counter in the process group's key-value store from a small thread; any
rank can ask which peers have not moved for ``stale_after`` seconds.  The engine front end checks
this *between* steps, before it launches kernels that wait on peers, so a lost rank is learned of on
the host and the step is refused with ``RankLost`` instead of running into device-side timeouts.

The reference detects a lost worker only through its control pipes (closed pipe => worker exits,
120 s socket poll timeout, include/b70/ipc_socket.hpp; a worker that throws leaves its loop,
grimoire.cpp:25114-25122) and has no recovery: a lost rank ends the server.  The same policy applies
here -- detection is fast and explicit, recovery is a restart.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Optional


class RankLost(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"ranks {sorted(ranks)} stopped responding")
        self.ranks = sorted(ranks)


class Heartbeat:
    """``store`` needs ``set(key, str)`` and ``get(key) -> bytes`` (c10d TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.5, stale_after: float = 3.0,
                 clock: Callable[[], float] = time.monotonic, prefix: str = "grm/hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.stale_after, self.clock, self.prefix = interval, stale_after, clock, prefix
        self._beat = 0
        self._seen: dict[int, tuple[int, float]] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beat()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def start(self) -> "Heartbeat":
        def run():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=run, name="grm-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def _read(self, r: int) -> int:
        try:
            return int(self.store.get(self._key(r)))
        except Exception:
            return -1

    def stale(self) -> list[int]:
        """Peers whose counter has not advanced for ``stale_after`` seconds (or never appeared)."""
        now = self.clock()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            last = self._seen.get(r)
            if last is None or v != last[0]:
                self._seen[r] = (v, now)
                if v < 0 and last is None:
                    self._seen[r] = (v, now)
                continue
            if now - last[1] >= self.stale_after:
                out.append(r)
        return out

    def check(self) -> None:
        dead = self.stale()
        if dead:
            raise RankLost(dead)
