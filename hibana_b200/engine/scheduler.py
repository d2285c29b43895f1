"""Continuous-batching scheduler with chunked prefill.

One `step()` = reap finished requests, admit from the FIFO queue while memory allows, then either a prefill
chunk (shortest-remaining-first under a token budget, with a bounded number of skips so nothing starves) followed
by `decode_steps_per_chunk` decode steps, or a decode step for everything running. A decode step that runs out of
KV memory retracts the newest request (it is re-admitted later and replays its emitted history).
Reference: hibana/engine/scheduler.py:29-294.
"""
from __future__ import annotations

import statistics
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Protocol, Sequence

from ..utils import nvtx
from .request import Request, State


class ExecutionBackend(Protocol):
    """What the scheduler needs from an executor (reference: hibana/engine/contracts.py:153-166)."""

    def validate_request(self, req: Request) -> None: ...
    def can_admit(self, req: Request) -> bool: ...
    def admit(self, req: Request) -> None: ...
    def prefill_batch(self, chunks: Sequence[tuple[Request, int]]) -> None: ...
    def decode_step(self, reqs: Sequence[Request]) -> None: ...
    def release(self, req: Request) -> None: ...
    def retract(self, req: Request) -> None: ...


@dataclass
class SchedulerConfig:
    prefill_chunk: int = 2048          # most tokens of one request per prefill forward
    prefill_budget: int = 4096         # most rows per prefill forward
    max_batch: int = 64
    max_queue: int = 256
    decode_steps_per_chunk: int = 1    # decode steps interleaved after every prefill chunk
    max_waits: int = 8                 # a prefilling request is skipped at most this many times


@dataclass
class Metrics:
    admitted: int = 0
    finished: int = 0
    cancelled: int = 0
    rejected: int = 0
    retractions: int = 0
    prefill_chunks: int = 0
    prefill_tokens: int = 0
    decode_steps: int = 0
    decode_tokens: int = 0
    steps: int = 0
    step_ms_sum: float = 0.0
    ttfts: deque = field(default_factory=lambda: deque(maxlen=2048))

    def latency_summary(self) -> dict:
        t = sorted(self.ttfts)
        if not t:
            return {"ttft_p50_ms": None, "ttft_p95_ms": None}
        return {"ttft_p50_ms": 1e3 * t[len(t) // 2], "ttft_p95_ms": 1e3 * t[min(len(t) - 1, int(len(t) * 0.95))]}

    def as_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if k != "ttfts"}
        d["avg_step_ms"] = self.step_ms_sum / self.steps if self.steps else 0.0
        d.update(self.latency_summary())
        return d


class QueueFull(Exception):
    pass


class Scheduler:
    def __init__(self, executor: ExecutionBackend, cfg: Optional[SchedulerConfig] = None):
        self.ex = executor
        self.cfg = cfg or SchedulerConfig()
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []         # admitted: prefilling or running, in admission order
        self.metrics = Metrics()
        self.sink = None                        # optional trace sink with .record(request)
        self.finished_hook = None               # optional callable(request) when a request leaves

    # ---- intake
    def submit(self, req: Request) -> Request:
        if len(self.waiting) >= self.cfg.max_queue:
            self.metrics.rejected += 1
            raise QueueFull(f"queue full ({self.cfg.max_queue})")
        try:
            self.ex.validate_request(req)
        except ValueError:
            self.metrics.rejected += 1
            raise
        self.waiting.append(req)
        return req

    def cancel(self, req: Request) -> None:
        req.cancel()

    def idle(self) -> bool:
        return not self.waiting and not self.active

    # ---- the step
    @nvtx.ranged("scheduler_step")
    def step(self) -> list[Request]:
        """Runs one scheduling step; returns the requests that produced tokens or finished in it."""
        t0 = time.perf_counter()
        touched: list[Request] = []
        self._reap(touched)
        self._admit()
        prefilling = [r for r in self.active if r.state == State.PREFILL]
        if prefilling:
            touched.extend(self._prefill_step(prefilling))
            for _ in range(self.cfg.decode_steps_per_chunk):
                touched.extend(self._decode())
        else:
            touched.extend(self._decode())
        self._reap(touched)
        self.metrics.steps += 1
        self.metrics.step_ms_sum += (time.perf_counter() - t0) * 1e3
        seen, out = set(), []
        for r in touched:
            if r.rid not in seen:
                seen.add(r.rid)
                out.append(r)
        return out

    def _reap(self, touched: list) -> None:
        for r in [r for r in self.active if r.done]:
            self.ex.release(r)
            self.active.remove(r)
            touched.append(r)
            if r.state == State.CANCELLED:
                self.metrics.cancelled += 1
            else:
                self.metrics.finished += 1
            if r.ttft is not None:
                self.metrics.ttfts.append(r.ttft)
            if self.sink is not None:
                self.sink.record(r)
            if self.finished_hook is not None:
                self.finished_hook(r)
        for r in [r for r in self.waiting if r.done]:
            self.waiting.remove(r)
            touched.append(r)
            self.metrics.cancelled += 1
            if self.finished_hook is not None:
                self.finished_hook(r)

    def _admit(self) -> None:
        """FIFO admission: the head of the queue must fit before anything behind it is considered."""
        while self.waiting and len(self.active) < self.cfg.max_batch:
            req = self.waiting[0]
            # KV slots the admitted requests still have to take for the rest of their prompts
            promised = sum(max(self._remaining_prefill(r), 0) for r in self.active if r.state == State.PREFILL)
            if not self._can_admit(req, promised):
                break
            try:
                self.ex.admit(req)
            except MemoryError:
                break
            self.waiting.popleft()
            self.active.append(req)
            self.metrics.admitted += 1

    def _can_admit(self, req: Request, promised: int) -> bool:
        try:
            return self.ex.can_admit(req, promised) if promised and self.active else self.ex.can_admit(req)
        except TypeError:               # executors of tests that take the request only
            return self.ex.can_admit(req)

    def _remaining_prefill(self, r: Request) -> int:
        total = r.total_len - (1 if r.output_ids else 0)
        return max(total - r.prefilled, 0)

    def _prefill_step(self, prefilling: list) -> list:
        """Shortest remaining first under the row budget; a request skipped `max_waits` times goes first."""
        order = sorted(prefilling, key=lambda r: (r.waits < self.cfg.max_waits, self._remaining_prefill(r)))
        budget = self.cfg.prefill_budget
        chunks = []
        for r in order:
            want = min(self._remaining_prefill(r), self.cfg.prefill_chunk)
            if want <= 0:
                continue
            if want > budget:
                if not chunks:
                    want = budget
                else:
                    r.waits += 1
                    continue
            chunks.append((r, want))
            r.waits = 0
            budget -= want
            if budget <= 0:
                break
        if not chunks:
            return []
        try:
            self.ex.prefill_batch(chunks)
        except MemoryError:
            victim = max((r for r, _ in chunks), key=lambda r: r.arrival)
            self._retract(victim)
            return []
        self.metrics.prefill_chunks += 1
        self.metrics.prefill_tokens += sum(c for _, c in chunks)
        return [r for r, _ in chunks]

    def _decode(self) -> list:
        running = [r for r in self.active if r.state == State.RUNNING and not r.done]
        while running:
            try:
                self.ex.decode_step(running)
                self.metrics.decode_steps += 1
                self.metrics.decode_tokens += len(running)
                return running
            except MemoryError:
                victim = max(running, key=lambda r: r.arrival)
                self._retract(victim)
                running.remove(victim)
        return []

    def _retract(self, req: Request) -> None:
        self.ex.retract(req)
        if req in self.active:
            self.active.remove(req)
        self.waiting.appendleft(req)
        self.metrics.retractions += 1

    # ---- failure
    def fail_all(self, reason: str) -> list[Request]:
        """Fails every request (engine failure): nothing of a failed forward is published to the cache."""
        out = []
        poison = getattr(getattr(self.ex, "state", None), "poison", None)
        if poison is not None:
            poison()
        for r in list(self.active):
            r.cacheable = False
            r.fail(reason)
            try:
                self.ex.release(r)
            except Exception:  # noqa: BLE001 - best effort while failing
                pass
            out.append(r)
        self.active.clear()
        for r in list(self.waiting):
            r.fail(reason)
            out.append(r)
        self.waiting.clear()
        return out
