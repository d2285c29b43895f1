"""Peer watchdog: every rank of a box publishes a heartbeat in the rendezvous store and watches the others'.

A rank that stops answering between steps (hung host thread, deadlocked collective, stopped process) cannot be
seen by its parent's `Popen.poll`, and the ranks that wait for it in a host broadcast would wait for ever. Each
rank therefore bumps `hb/<rank>` in the store every `interval` seconds from a daemon thread and calls `on_dead`
with the silent ranks once a peer's counter has not moved for `timeout` seconds; the engine fails its tickets and
exits non-zero, which makes the supervisor restart the whole group (launch/supervisor.py). Nothing here touches a
GPU: detection is host-side by construction. Reference: hibana/distributed.py:70-108 (peer watchdog),
docs/tensor-parallel.md:32 (rank SIGKILL -> serving again).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Optional, Sequence


class PeerWatchdog:
    def __init__(self, store, rank: int, world: int, *, interval: float = 1.0, timeout: float = 10.0,
                 on_dead: Optional[Callable[[Sequence[int]], None]] = None,
                 clock: Callable[[], float] = time.monotonic, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.on_dead, self.clock, self.prefix = interval, timeout, on_dead, clock, prefix
        self.count = 0
        now = clock()
        self.last_value = {r: None for r in range(world) if r != rank}
        self.last_change = {r: now for r in range(world) if r != rank}
        self.dead: list[int] = []
        self._stop = threading.Event()
        self.thread: Optional[threading.Thread] = None

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self.count += 1
        self.store.set(self._key(self.rank), str(self.count))

    def check(self) -> list[int]:
        """Ranks whose heartbeat has not moved for `timeout` seconds (a rank that never wrote one counts from the
        watchdog's start)."""
        now = self.clock()
        dead = []
        for r in self.last_value:
            val = None
            try:
                if self.store.check([self._key(r)]):
                    val = self.store.get(self._key(r))
            except Exception:  # noqa: BLE001 - a store that went away (rank 0 hosts it) is a dead peer as well
                val = None
            if val is not None and val != self.last_value[r]:
                self.last_value[r], self.last_change[r] = val, now
            elif now - self.last_change[r] > self.timeout:
                dead.append(r)
        self.dead = dead
        return dead

    def start(self) -> "PeerWatchdog":
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001 - the store host died
                    if self.on_dead is not None:
                        self.on_dead([0])
                    return
                dead = self.check()
                if dead and self.on_dead is not None:
                    self.on_dead(dead)
                    return
        self.beat()
        self.thread = threading.Thread(target=loop, name="hibana-watchdog", daemon=True)
        self.thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
