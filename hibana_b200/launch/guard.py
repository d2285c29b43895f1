"""Memory guard thread: when free host memory stays under half the floor for 3 samples (2 s apart) the engine is
asked to stop (SIGTERM), and killed 15 s later if still alive. Reference: hibana/launch/guard.py:1-98."""
from __future__ import annotations

import os
import signal
import threading
import time
from typing import Callable, Optional


def host_free_gib() -> float:
    try:
        import psutil
        return psutil.virtual_memory().available / (1 << 30)
    except Exception:  # noqa: BLE001
        return float("inf")


class MemoryGuard:
    def __init__(self, floor_gib: float, pid: Optional[int] = None, probe: Callable[[], float] = host_free_gib,
                 interval: float = 2.0, samples: int = 3, kill_after: float = 15.0,
                 send: Callable[[int, int], None] = os.kill):
        self.floor, self.pid = floor_gib, pid or os.getpid()
        self.probe, self.interval, self.samples, self.kill_after, self.send = probe, interval, samples, kill_after, send
        self.low = 0
        self.fired = False
        self._stop = threading.Event()
        self.thread: Optional[threading.Thread] = None

    def sample(self) -> bool:
        """One observation; returns True when the guard fires."""
        self.low = self.low + 1 if self.probe() < self.floor / 2 else 0
        if self.low >= self.samples and not self.fired:
            self.fired = True
            self.send(self.pid, signal.SIGTERM)
            return True
        return False

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            if self.sample():
                if not self._stop.wait(self.kill_after):
                    try:
                        self.send(self.pid, signal.SIGKILL)
                    except ProcessLookupError:
                        pass
                return

    def start(self) -> "MemoryGuard":
        self.thread = threading.Thread(target=self._run, name="hibana-guard", daemon=True)
        self.thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
