"""Engine loop: one engine thread owns the scheduler and everything below it; other threads only enqueue.

`submit` returns a `Ticket` whose queue receives `("tokens", [ids])` events and finally `("done", reason)` or
`("error", message)`. With tensor parallelism rank 0 owns the inbox and broadcasts the commands it applied at
every publish point, so all ranks step their schedulers identically; a failure fails every ticket and marks the
engine unhealthy. With data-parallel replicas (`dp`, an engine/dp.py Lockstep) rank 0 still owns HTTP and the
inbox but every request has ONE owner: rank 0 picks the replica (least outstanding work, conversations stay with
their cached prefix), commands and generated tokens travel with the lockstep rounds, and the replicas schedule
independently. A replica that is itself a tensor-parallel group has both: its leader joins the rounds and
broadcasts what it applies to its followers. Reference: hibana/engine/loop.py:47-320.
"""
from __future__ import annotations

import dataclasses
import itertools
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

from .request import Request, SamplingParams
from .scheduler import QueueFull, Scheduler


@dataclass
class Ticket:
    tid: int
    request: Optional[Request] = None
    events: "queue.Queue" = field(default_factory=queue.Queue)
    notify: Optional[Callable[[], None]] = None     # e.g. loop.call_soon_threadsafe wakeup for asyncio consumers
    cursor: int = 0
    closed: bool = False

    def put(self, item) -> None:
        self.events.put(item)
        if self.notify is not None:
            self.notify()


class EngineUnavailable(RuntimeError):
    pass


class _Load:
    """Outstanding requests of one replica, as the router's `stats()` source."""

    def __init__(self):
        self.n = 0

    def stats(self) -> dict:
        return {"running": self.n, "waiting": 0}


class EngineLoop:
    def __init__(self, scheduler: Scheduler, channel=None, rank: int = 0, idle_sleep: float = 0.002, dp=None):
        self.sched = scheduler
        self.channel = channel          # lockstep command channel (None = single rank)
        self.dp = dp                    # engine/dp.py Lockstep of data-parallel replicas (None = one replica)
        self.rank = rank
        self._mail: list = []           # commands (from rank 0) and outputs (to rank 0) received in rounds
        self._router = None
        self._outstanding: dict[int, int] = {}    # rank 0: tid -> owner of every unfinished remote or local request
        if dp is not None:
            dp.on_items = lambda src, items: self._mail.extend((src, i) for i in items)
            if rank == 0:
                from .dp import ReplicaSet
                loads = [_Load() for _ in range(dp.world)]
                self._router = ReplicaSet(loads)
        self.idle_sleep = idle_sleep
        self.inbox: "queue.Queue" = queue.Queue()
        self.tickets: dict[int, Ticket] = {}
        self._by_rid: dict[int, Ticket] = {}
        self._ids = itertools.count(1)
        self.healthy = True
        self.grammars = None      # engine.grammar.Grammars (or a factory); needed on every rank when a channel is set
        self.failure: Optional[str] = None
        self.stopping = False
        self.draining = False
        self.thread: Optional[threading.Thread] = None
        self.steps = 0
        self._applied: list = []

    # ---- any thread
    def start(self) -> "EngineLoop":
        self.thread = threading.Thread(target=self._run, name="hibana-engine", daemon=True)
        self.thread.start()
        return self

    def submit(self, prompt_ids, params: SamplingParams, *, eos_id=None, media=None, constraint=None,
               notify=None) -> Ticket:
        if not self.healthy:
            raise EngineUnavailable(self.failure or "engine failed")
        if self.draining or self.stopping:
            raise EngineUnavailable("engine is shutting down")
        if self.inbox.qsize() + len(self.sched.waiting) >= self.sched.cfg.max_queue:
            raise QueueFull("queue full")
        t = Ticket(next(self._ids), notify=notify)
        self.tickets[t.tid] = t
        constraint = constraint if constraint is not None else params.constraint
        if constraint is not None and (self.channel is not None or self.dp is not None):
            # a compiled grammar does not pickle: other ranks get its source and compile it again (self.grammars)
            constraint = ("source", constraint.kind, constraint.source, constraint.think_end)
            params = dataclasses.replace(params, constraint=None)
        self.inbox.put(("submit", t.tid, list(prompt_ids), params, eos_id, media, constraint))
        return t

    def cancel(self, ticket: Ticket) -> None:
        self.inbox.put(("cancel", ticket.tid))

    def drain(self, timeout: float = 30.0) -> bool:
        """Stops intake and waits until every admitted request has finished."""
        self.draining = True
        end = time.monotonic() + timeout
        while time.monotonic() < end:
            if self.sched.idle() and self.inbox.empty():
                return True
            time.sleep(0.01)
        return False

    def stop(self, timeout: float = 10.0) -> None:
        self.stopping = True
        self.inbox.put(("stop",))
        if self.thread is not None:
            self.thread.join(timeout)

    def stats(self) -> dict:
        d = self.sched.metrics.as_dict()
        d.update({"healthy": self.healthy, "queued": len(self.sched.waiting), "active": len(self.sched.active),
                  "engine_steps": self.steps})
        ex_state = getattr(self.sched.ex, "state", None)
        if ex_state is not None:
            d["cache"] = ex_state.stats()
        return d

    # ---- engine thread
    def _apply(self, cmd) -> None:
        kind = cmd[0]
        if kind == "submit":
            _, tid, ids, params, eos_id, media, constraint = cmd
            ticket = self.tickets.get(tid)
            if ticket is None and self.dp is not None and self.rank != 0:
                ticket = self.tickets[tid] = Ticket(tid)          # stand-in: its events go to rank 0 in rounds
            if isinstance(constraint, tuple):       # rebuilt on every rank from the broadcast source
                gr = self.grammars() if callable(self.grammars) else self.grammars
                constraint = gr.recompile(*constraint[1:]) if gr is not None else None
            if constraint is not None and params.constraint is not constraint:
                params = dataclasses.replace(params, constraint=constraint)
            req = Request(prompt_ids=ids, params=params, eos_id=eos_id, media=media)
            try:
                self.sched.submit(req)
            except (ValueError, QueueFull) as e:
                if ticket is not None:
                    if self.dp is not None and self.rank != 0:
                        self.dp.post(("out", tid, [], None, str(e)))
                        self.tickets.pop(tid, None)
                    else:
                        ticket.put(("error", str(e)))
                        self._finished(tid)
                    ticket.closed = True
                return
            if ticket is not None:
                ticket.request = req
                self._by_rid[req.rid] = ticket
        elif kind == "cancel":
            ticket = self.tickets.get(cmd[1])
            if ticket is not None and ticket.request is not None:
                self.sched.cancel(ticket.request)
        elif kind == "stop":
            self.stopping = True
        elif kind == "failed":          # the leader of this tensor-parallel group gave up
            raise RuntimeError(f"group leader failed: {cmd[1]}")

    def _gather_commands(self) -> list:
        cmds = []
        while True:
            try:
                cmds.append(self.inbox.get_nowait())
            except queue.Empty:
                break
        return cmds

    def _publish_commands(self, cmds: list) -> list:
        """Rank 0 broadcasts what it is about to apply; other ranks receive the same list."""
        if self.channel is None:
            return cmds
        if self.rank == 0:
            # tickets and notifiers stay local: ship only plain data
            self.channel.broadcast(cmds)
            return cmds
        return self.channel.broadcast(None)

    def _deliver(self, touched) -> None:
        for req in touched:
            ticket = self._by_rid.get(req.rid)
            if ticket is None or ticket.closed:
                continue
            new = req.output_ids[ticket.cursor:]
            if self.dp is not None and self.rank != 0:      # the ticket's consumer lives on rank 0
                ticket.cursor += len(new)
                if new or req.done:
                    self.dp.post(("out", ticket.tid, list(new), req.finish_reason if req.done else None, None))
                if req.done:
                    ticket.closed = True
                    self._by_rid.pop(req.rid, None)
                    self.tickets.pop(ticket.tid, None)
                continue
            if new:
                ticket.cursor += len(new)
                ticket.put(("tokens", list(new)))
            if req.done:
                ticket.put(("done", req.finish_reason))
                ticket.closed = True
                self._by_rid.pop(req.rid, None)
                self.tickets.pop(ticket.tid, None)
                self._finished(ticket.tid)

    def _fail(self, message: str) -> None:
        self.healthy = False
        self.failure = message
        for req in self.sched.fail_all(message):
            ticket = self._by_rid.pop(req.rid, None)
            if ticket is not None and not ticket.closed:
                ticket.put(("error", message))
                ticket.closed = True
        for ticket in list(self.tickets.values()):
            if not ticket.closed:
                ticket.put(("error", message))
                ticket.closed = True
        self.tickets.clear()

    # ---- data-parallel replicas
    def _route(self, cmds: list) -> list:
        """Rank 0: gives every submit an owner and posts the commands of other owners; returns its own."""
        mine = []
        for c in cmds:
            if c[0] == "submit":
                owner = self._router.pick(c[2])
                self._router.loops[owner].n += 1
                self._outstanding[c[1]] = owner
                if owner == 0:
                    mine.append(c)
                else:
                    self.dp.post(("cmd", owner, c))
            elif c[0] == "cancel":
                owner = self._outstanding.get(c[1], 0)
                if owner == 0:
                    mine.append(c)
                else:
                    self.dp.post(("cmd", owner, c))
            else:                                   # stop: everyone
                self.dp.post(("cmd", -1, c))
                mine.append(c)
        return mine

    def _finished(self, tid: int) -> None:
        owner = self._outstanding.pop(tid, None)
        if owner is not None and self._router is not None:
            self._router.loops[owner].n -= 1

    def _take_mail(self) -> list:
        """Commands addressed to this rank; on rank 0 also delivers the other replicas' outputs to the tickets."""
        mail, self._mail = self._mail, []
        cmds = []
        for _src, item in mail:
            if item[0] == "cmd":
                if item[1] in (-1, self.rank):
                    cmds.append(item[2])
            elif item[0] == "out" and self.rank == 0:
                _, tid, tokens, done, error = item
                ticket = self.tickets.get(tid)
                if ticket is None or ticket.closed:
                    continue
                if tokens:
                    ticket.put(("tokens", tokens))
                if error is not None or done is not None:
                    ticket.put(("error", error) if error is not None else ("done", done))
                    ticket.closed = True
                    self.tickets.pop(tid, None)
                    self._finished(tid)
            elif item[0] == "failed":
                from .dp import ReplicaFailed
                raise ReplicaFailed(f"replica {_src} failed: {item[1]}")
        return cmds

    def _run_dp(self) -> None:
        from .dp import LEAVING, RUNNING
        ex = self.sched.ex
        try:
            while True:
                cmds = self._route(self._gather_commands()) if self.rank == 0 else []
                cmds = cmds + self._take_mail()
                if self.channel is not None:
                    # this replica is a tensor-parallel group: its followers apply the same commands and so take
                    # the same steps. `stop` reaches them when this loop ends, not when it is asked to.
                    self.channel.broadcast([c for c in cmds if c[0] != "stop"])
                for c in cmds:
                    self._apply(c)
                if self.sched.idle():
                    states = ex.idle_round(LEAVING if self.stopping else RUNNING)
                    if self.stopping and all(s == LEAVING for s in states):
                        if self.channel is not None:
                            self.channel.broadcast([("stop",)])
                        break
                    if 1 not in states and not self._mail:
                        time.sleep(self.idle_sleep)
                    continue
                touched = self.sched.step()
                self.steps += 1
                self._deliver(touched)
        except Exception as e:  # noqa: BLE001 - every failure takes the engine down cleanly
            from .dp import ReplicaFailed
            try:
                if self.channel is not None:
                    self.channel.broadcast([("failed", f"{type(e).__name__}: {e}")])
                if not isinstance(e, ReplicaFailed) and not self.dp.broken:
                    # this replica's own failure: one last round carries the news, so the others stop at their next
                    # round instead of waiting for the control timeout. (A replica that stops because another one
                    # failed joins no further round: nobody would be there.)
                    self.dp.post(("failed", f"{type(e).__name__}: {e}"))
                    self.dp.round(LEAVING)
            except Exception:  # noqa: BLE001 - best effort: the peers' timeouts cover a round nobody joins
                pass
            finally:
                self._fail(f"{type(e).__name__}: {e}")

    def _run(self) -> None:
        if self.dp is not None:
            return self._run_dp()
        try:
            while True:
                cmds = self._publish_commands(self._gather_commands())
                for c in cmds:
                    self._apply(c)
                if self.stopping:
                    break
                if self.sched.idle():
                    if self.channel is None:
                        time.sleep(self.idle_sleep)
                    continue
                touched = self.sched.step()
                self.steps += 1
                self._deliver(touched)
        except Exception as e:  # noqa: BLE001 - every failure takes the engine down cleanly
            self._fail(f"{type(e).__name__}: {e}")
