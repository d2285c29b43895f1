"""Rank supervisor for one box: spawns one engine process per GPU, watches them, restarts the whole group when any
rank dies (at most 5 restarts in 600 s). A dead rank is noticed by its parent through `Popen.poll` (no network
keepalive is needed inside one host); the prefix cache survives restarts through the SSD tier.
Reference: hibana/launch/tp.py (Pair, restart loop 5 in 600 s) and hibana/distributed.py:70-108 (peer watchdog).
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from typing import Callable, Optional, Sequence

MAX_RESTARTS, WINDOW_S = 5, 600.0


class RankGroup:
    def __init__(self, world: int, argv: Sequence[str], *, master_port: int = 29500, env: Optional[dict] = None,
                 spawn: Callable = subprocess.Popen):
        self.world, self.argv, self.port, self.spawn = world, list(argv), master_port, spawn
        self.env = dict(os.environ if env is None else env)
        self.procs: list = []

    def start(self) -> None:
        self.procs = []
        for rank in range(self.world):
            env = dict(self.env, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(self.world),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(self.port))
            self.procs.append(self.spawn(self.argv, env=env))

    def poll(self) -> Optional[tuple[int, int]]:
        """(rank, exit code) of the first rank that has exited, else None."""
        for rank, p in enumerate(self.procs):
            code = p.poll()
            if code is not None:
                return rank, code
        return None

    def stop(self, grace: float = 10.0) -> None:
        for p in self.procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        end = time.monotonic() + grace
        for p in self.procs:
            while p.poll() is None and time.monotonic() < end:
                time.sleep(0.05)
            if p.poll() is None:
                p.kill()


class Supervisor:
    def __init__(self, group: RankGroup, *, clock: Callable[[], float] = time.monotonic,
                 sleep: Callable[[float], None] = time.sleep, log: Callable[[str], None] = print):
        self.group, self.clock, self.sleep, self.log = group, clock, sleep, log
        self.restarts: list[float] = []
        self.stopping = False

    def allowed(self) -> bool:
        now = self.clock()
        self.restarts = [t for t in self.restarts if now - t < WINDOW_S]
        return len(self.restarts) < MAX_RESTARTS

    def run(self, poll_interval: float = 0.5) -> int:
        """Runs until a clean exit (all ranks 0), a stop request, or the restart budget is spent."""
        self.group.start()
        while True:
            dead = self.group.poll()
            if dead is None:
                if self.stopping:
                    self.group.stop()
                    return 0
                self.sleep(poll_interval)
                continue
            rank, code = dead
            if code == 0 and all(p.poll() == 0 for p in self.group.procs):
                return 0
            self.log(f"rank {rank} exited with {code}; stopping the group")
            self.group.stop()
            if self.stopping:
                return 0
            if not self.allowed():
                self.log("restart budget spent (5 in 600 s)")
                return 1
            self.restarts.append(self.clock())
            self.log(f"restarting the group (restart {len(self.restarts)})")
            self.group.start()


def engine_argv(extra: Sequence[str]) -> list[str]:
    return [sys.executable, "-m", "hibana_b200", "engine", *extra]
