"""Data-parallel replicas: several engines (one per GPU or per tensor-parallel group) behind one front end.

`ReplicaSet` routes every new request to the replica with the least outstanding work, keeps follow-up turns of a
conversation on the replica whose prefix cache already holds the conversation (prefix affinity by a hash of the
leading tokens), and drains / reports per replica. With expert parallelism across the replicas (DP attention + EP
experts) the replicas additionally step in lockstep: `lockstep_plan` tells every replica, from the all-gathered
"do I have work" bits, whether the step runs and whether it must run with an empty batch (a rank without requests
still has to take part in the all-to-all of every MoE layer). The reference serves one engine per process
(hibana/engine/loop.py); data parallelism is new here.
"""
from __future__ import annotations

import hashlib
import threading
from typing import Any, Callable, Optional, Sequence

RUNNING, FORWARD, LEAVING = 0, 1, 2      # what a rank posts in a round


class ReplicaSet:
    def __init__(self, loops: Sequence[Any], affinity_tokens: int = 256, affinity_slack: int = 4):
        """`loops`: objects with submit(request) -> ticket, stats() -> {"running": int, "waiting": int}."""
        assert loops
        self.loops = list(loops)
        self.affinity_tokens, self.affinity_slack = affinity_tokens, affinity_slack
        self._home: dict[bytes, int] = {}
        self.routed = [0] * len(self.loops)

    def _load(self, i: int) -> int:
        st = self.loops[i].stats()
        return int(st.get("running", 0)) + int(st.get("waiting", 0))

    def _key(self, prompt_ids: Sequence[int]) -> Optional[bytes]:
        if len(prompt_ids) < self.affinity_tokens:
            return None
        head = prompt_ids[:self.affinity_tokens]
        return hashlib.blake2b(b"".join(int(t).to_bytes(8, "little", signed=True) for t in head), digest_size=16).digest()

    def pick(self, prompt_ids: Sequence[int]) -> int:
        loads = [self._load(i) for i in range(len(self.loops))]
        best = min(range(len(loads)), key=lambda i: (loads[i], i))
        key = self._key(prompt_ids)
        if key is not None:
            home = self._home.get(key)
            # stay with the cached prefix unless that replica is clearly busier than the idlest one
            if home is not None and loads[home] <= loads[best] + self.affinity_slack:
                best = home
            self._home[key] = best
            if len(self._home) > 65536:
                self._home.pop(next(iter(self._home)))
        return best

    def submit(self, request) -> Any:
        i = self.pick(request.prompt_ids)
        self.routed[i] += 1
        return self.loops[i].submit(request)

    def stats(self) -> dict:
        per = [loop.stats() for loop in self.loops]
        return {"replicas": len(per), "routed": list(self.routed),
                "running": sum(int(p.get("running", 0)) for p in per),
                "waiting": sum(int(p.get("waiting", 0)) for p in per), "per_replica": per}

    def drain(self) -> None:
        for loop in self.loops:
            if hasattr(loop, "drain"):
                loop.drain()


def lockstep_plan(has_work: Sequence[bool]) -> tuple[bool, list[bool]]:
    """(run the step at all, per replica: run with an empty batch). Expert-parallel replicas only skip a step when
    nobody has work."""
    if not any(has_work):
        return False, [False] * len(has_work)
    return True, [not w for w in has_work]


class ReplicaFailed(RuntimeError):
    """Another replica reported that it gave up (its message arrived with a round)."""


class Lockstep:
    """Round protocol of data-parallel ranks that share expert-parallel layers.

    Ranks schedule their own requests, so their steps differ (one prefills and decodes while another only
    decodes, a third is idle), but every forward pass runs the all-to-all of every MoE layer and needs all ranks
    in it. Ranks therefore align FORWARDS, not steps: before each forward a rank posts FORWARD in a round; a rank
    with nothing to run posts RUNNING (or LEAVING once it has been told to stop and has drained) and, when any
    other rank posted FORWARD, runs the model on an empty batch. A round is one all-gather of small host objects
    over the control group; it also carries the messages of the data-parallel front end (commands from rank 0,
    generated tokens back to it), so steady decoding costs one host collective per step. The loop ends in the
    first round in which every rank posts LEAVING. The reference steps identical schedulers from broadcast
    commands (hibana/engine/loop.py:163-182); ranks with different work are new here.
    """

    def __init__(self, allgather: Callable[[Any], list], rank: int, world: int):
        self.allgather, self.rank, self.world = allgather, rank, world
        self.outbox: list = []
        self.on_items: Optional[Callable[[int, list], None]] = None
        self.rounds = self.forward_rounds = self.empty_forwards = 0
        self.broken = False          # a round's all-gather raised (a replica stopped answering): no more rounds

    def post(self, item) -> None:
        """Queues a picklable message for every other rank; it travels with the next round."""
        self.outbox.append(item)

    def round(self, state: int) -> list:
        mine, self.outbox = (int(state), self.outbox), []
        try:
            got = self.allgather(mine)
        except BaseException:
            self.broken = True
            raise
        self.rounds += 1
        states = [g[0] for g in got]
        self.forward_rounds += FORWARD in states
        if self.on_items is not None:
            for src, (_, items) in enumerate(got):
                if items and src != self.rank:
                    self.on_items(src, items)
        return states


class GroupAllGather:
    """`Lockstep` transport over a torch.distributed group (the CPU control group of the ranks)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group)

    def __call__(self, obj) -> list:
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self.group)
        return out


class ThreadAllGather:
    """`Lockstep` transport between threads of one process (tests; replicas that share a GPU never use
    kernels that wait on one another)."""

    def __init__(self, world: int, timeout: float = 60.0):
        self.world, self.timeout = world, timeout
        self.slots: list = [None] * world
        self.barrier = threading.Barrier(world)

    def view(self, rank: int) -> Callable[[Any], list]:
        def gather(obj):
            self.slots[rank] = obj
            self.barrier.wait(self.timeout)
            out = list(self.slots)
            self.barrier.wait(self.timeout)
            return out
        return gather
