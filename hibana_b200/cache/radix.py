"""Radix prefix cache over token ids, holding KV slots and recurrent-state snapshots.

Every node stores a run of tokens with the KV slot of each token; a node may carry one `Snapshot` (recurrent state
slot valid exactly at the node's end). Protection is by locks only: `lock_ref(n)` counts locks at n or below
(keeps n's KV), `state_lock_ref(n)` counts locks on n itself (keeps n's snapshot). Nodes split and prune, never
merge. Evictable totals are maintained incrementally so admission can budget without evicting. Logical ticks
(not wall time) order evictions, so tensor-parallel ranks choose alike.
Reference: hibana/cache/radix.py:126-818 and docs/cache_design.md:73-170.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence


@dataclass
class Snapshot:
    slot: int                 # state-pool slot holding the recurrent state after `position` tokens
    position: int
    spare: bool = False       # probationary (evicted before non-spare ones)
    tick: int = 0
    auxiliary: Any = None     # drafter metadata


class Node:
    __slots__ = ("tokens", "slots", "children", "parent", "lock_ref", "state_lock_ref", "snapshot", "tick",
                 "on_ssd", "depth")

    def __init__(self, tokens: list, slots: list, parent: Optional["Node"]):
        self.tokens, self.slots, self.parent = tokens, slots, parent
        self.children: dict[int, Node] = {}
        self.lock_ref = 0
        self.state_lock_ref = 0
        self.snapshot: Optional[Snapshot] = None
        self.tick = 0
        self.on_ssd = False
        self.depth = (parent.depth + len(parent.tokens)) if parent is not None else 0

    @property
    def end(self) -> int:
        return self.depth + len(self.tokens)

    def path_slots(self) -> list:
        parts, n = [], self
        while n is not None:
            parts.append(n.slots)
            n = n.parent
        out: list = []
        for p in reversed(parts):
            out.extend(p)
        return out


@dataclass
class TreeLock:
    node: Node
    released: bool = False


@dataclass
class Match:
    node: Node                 # deepest node fully or partly matched (after a split it ends at `length`)
    length: int                # matched tokens
    slots: list                # KV slots of the matched tokens
    state_node: Optional[Node]  # deepest node on the path with a snapshot
    state_length: int          # its end position (0 = none)
    branch_at: int = 0         # where the query left the existing tree (a snapshot here helps the next request)


class RadixCache:
    def __init__(self, free_kv: Callable[[Sequence[int]], None], free_state: Optional[Callable[[int], None]] = None,
                 needs_state: bool = False):
        self.root = Node([], [], None)
        self.root.lock_ref = 1   # never evicted
        self._free_kv, self._free_state = free_kv, free_state
        self.needs_state = needs_state
        self._tick = 0
        self.size = 0                    # tokens held
        self.evictable_size = 0          # tokens in nodes with lock_ref == 0
        self.snapshots = 0
        self.state_evictable = 0         # snapshots on nodes with state_lock_ref == 0
        self.hits = self.misses = self.full_reprefills = 0
        self.ssd_hook = None             # called before KV of a node is freed (SSD tier backup bookkeeping)

    # ---- helpers
    def _touch(self, node: Node) -> None:
        self._tick += 1
        while node is not None:
            node.tick = self._tick
            if node.snapshot is not None:
                node.snapshot.tick = self._tick
            node = node.parent

    def _walk(self, tokens: Sequence[int]):
        """Yields (node, matched_in_node) along the path; stops at the first partial / missing edge."""
        node, i = self.root, 0
        n = len(tokens)
        while i < n:
            child = node.children.get(tokens[i])
            if child is None:
                return
            m, lim = 0, min(len(child.tokens), n - i)
            ct = child.tokens
            while m < lim and ct[m] == tokens[i + m]:
                m += 1
            yield child, m
            if m < len(ct):
                return
            node, i = child, i + m

    def _split(self, node: Node, at: int) -> Node:
        """Splits `node` after `at` tokens; returns the upper part (which keeps the parent link)."""
        assert 0 < at < len(node.tokens)
        upper = Node(node.tokens[:at], node.slots[:at], node.parent)
        upper.lock_ref = node.lock_ref          # every lock below still passes through the upper part
        upper.tick = node.tick
        upper.on_ssd = node.on_ssd
        node.parent.children[upper.tokens[0]] = upper
        node.tokens, node.slots = node.tokens[at:], node.slots[at:]
        node.parent = upper
        node.depth = upper.end
        upper.children[node.tokens[0]] = node
        if upper.lock_ref == 0:
            pass  # evictable totals unchanged: the same tokens, now in two unlocked nodes
        return upper

    # ---- queries
    def match(self, tokens: Sequence[int], split: bool = True) -> Match:
        """Longest cached prefix of `tokens`. With split=True a partly matched node is split at the match point
        so the result ends on a node boundary (needed before locking); split=False leaves the tree untouched."""
        node, length, slots = self.root, 0, []
        state_node, state_len = None, 0
        for child, m in self._walk(tokens):
            if m < len(child.tokens):
                if m == 0:
                    break
                if split:
                    child = self._split(child, m)
                    node = child
                    slots.extend(child.slots)
                else:
                    slots.extend(child.slots[:m])
                    node = child
                length += m
                if split and child.snapshot is not None:
                    state_node, state_len = child, child.end
                break
            node = child
            slots.extend(child.slots)
            length += m
            if child.snapshot is not None:
                state_node, state_len = child, child.end
        if length:
            self.hits += 1
            if split:
                self._touch(node)
        else:
            self.misses += 1
        return Match(node, length, slots, state_node, state_len, branch_at=length)

    def usable(self, m: Match) -> tuple[Node, int]:
        """(node, length) a request can actually resume from: the KV match, or the deepest snapshot when the model
        has recurrent state."""
        if not self.needs_state:
            return m.node, m.length
        if m.state_node is None:
            if m.length:
                self.full_reprefills += 1
            return self.root, 0
        return m.state_node, m.state_length

    # ---- locks
    def lock(self, node: Node) -> TreeLock:
        if node.state_lock_ref == 0 and node.snapshot is not None:
            self.state_evictable -= 1
        node.state_lock_ref += 1
        n = node
        while n is not None and n is not self.root:
            if n.lock_ref == 0:
                self.evictable_size -= len(n.tokens)
            n.lock_ref += 1
            n = n.parent
        return TreeLock(node)

    def unlock(self, lock: Optional[TreeLock]) -> None:
        if lock is None or lock.released:
            return
        lock.released = True
        node = lock.node
        node.state_lock_ref -= 1
        assert node.state_lock_ref >= 0
        if node.state_lock_ref == 0 and node.snapshot is not None:
            self.state_evictable += 1
        n = node
        while n is not None and n is not self.root:
            n.lock_ref -= 1
            assert n.lock_ref >= 0
            if n.lock_ref == 0:
                self.evictable_size += len(n.tokens)
            n = n.parent

    def move_lock(self, lock: TreeLock, node: Node) -> TreeLock:
        """Moves a request's lock to a deeper node (after a prefill chunk was inserted)."""
        new = self.lock(node)
        self.unlock(lock)
        return new

    # ---- insertion
    def insert(self, tokens: Sequence[int], slots: Sequence[int], start: int = 0) -> tuple[Node, int]:
        """Inserts tokens[0:len] whose KV slots are `slots`; positions < `start` are known to be in the tree with
        these very slots. Returns (deepest node reached, adopted_upto): slots of positions [start, adopted_upto)
        now belong to the tree. Adoption stops where the tree already holds other slots for the same tokens."""
        assert len(tokens) == len(slots)
        node, i, n = self.root, 0, len(tokens)
        adopted = start
        while i < n:
            child = node.children.get(tokens[i])
            if child is None:
                if i >= start:
                    new = Node(list(tokens[i:]), list(slots[i:]), node)
                    node.children[tokens[i]] = new
                    self.size += n - i
                    self.evictable_size += n - i
                    adopted, node = n, new
                break
            if i >= start:
                break   # someone else already cached these tokens with other slots: the caller keeps its copy
            ct = child.tokens
            m, lim = 0, min(len(ct), n - i)
            while m < lim and ct[m] == tokens[i + m]:
                m += 1
            if m == 0:
                break
            if m < len(ct):
                child = self._split(child, m)
            node, i = child, i + m
        self._touch(node)
        return node, adopted

    def set_snapshot(self, node: Node, snap: Snapshot) -> Optional[Snapshot]:
        """Attaches a snapshot to a node whose end equals snap.position; returns a replaced snapshot (to free)."""
        assert node.end == snap.position, (node.end, snap.position)
        old = node.snapshot
        if old is None:
            self.snapshots += 1
            if node.state_lock_ref == 0:
                self.state_evictable += 1
        self._tick += 1
        snap.tick = self._tick
        node.snapshot = snap
        return old

    # ---- eviction
    def _leaves(self):
        stack = [self.root]
        while stack:
            n = stack.pop()
            if not n.children and n is not self.root:
                yield n
            stack.extend(n.children.values())

    def _drop_snapshot(self, node: Node) -> None:
        if node.snapshot is None:
            return
        if node.state_lock_ref == 0:
            self.state_evictable -= 1
        self.snapshots -= 1
        if self._free_state is not None:
            self._free_state(node.snapshot.slot)
        node.snapshot = None

    def evict(self, tokens_needed: int) -> int:
        """Frees KV of unlocked leaves in LRU order (copies already on SSD first) until `tokens_needed` tokens
        were freed or nothing evictable is left. Returns tokens freed."""
        freed = 0
        while freed < tokens_needed:
            cands = [n for n in self._leaves() if n.lock_ref == 0 and n.state_lock_ref == 0]
            if not cands:
                break
            cands.sort(key=lambda n: (not n.on_ssd, n.tick))
            for leaf in cands:
                if freed >= tokens_needed:
                    break
                if leaf.children:
                    continue
                if self.ssd_hook is not None:
                    self.ssd_hook(leaf)
                self._drop_snapshot(leaf)
                self._free_kv(leaf.slots)
                freed += len(leaf.tokens)
                self.size -= len(leaf.tokens)
                self.evictable_size -= len(leaf.tokens)
                del leaf.parent.children[leaf.tokens[0]]
                leaf.parent = None
        return freed

    def evict_snapshots(self, count: int) -> int:
        """Frees up to `count` unlocked snapshots, spare ones first, then least recently used."""
        cands = []
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n.snapshot is not None and n.state_lock_ref == 0:
                cands.append(n)
            stack.extend(n.children.values())
        cands.sort(key=lambda n: (not n.snapshot.spare, n.snapshot.tick))
        done = 0
        for n in cands[:count]:
            self._drop_snapshot(n)
            done += 1
        return done

    def flush(self) -> int:
        """Drops everything that is not locked. Returns tokens freed."""
        self.evict_snapshots(self.snapshots)
        return self.evict(self.size)

    # ---- invariants and stats
    def check(self) -> None:
        size = evictable = snaps = state_ev = 0
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n is not self.root:
                assert n.tokens and len(n.tokens) == len(n.slots)
                assert n.parent.children[n.tokens[0]] is n
                assert n.depth == n.parent.end
                size += len(n.tokens)
                if n.lock_ref == 0:
                    evictable += len(n.tokens)
                assert n.lock_ref == n.state_lock_ref + sum(c.lock_ref for c in n.children.values()), \
                    "lock_ref(n) == state_lock_ref(n) + sum lock_ref(child)"
            if n.snapshot is not None:
                assert n.snapshot.position == n.end
                snaps += 1
                if n.state_lock_ref == 0:
                    state_ev += 1
            stack.extend(n.children.values())
        assert size == self.size, (size, self.size)
        assert evictable == self.evictable_size, (evictable, self.evictable_size)
        assert snaps == self.snapshots and state_ev == self.state_evictable

    def all_slots(self) -> list:
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            out.extend(n.slots)
            stack.extend(n.children.values())
        return out

    def stats(self) -> dict:
        return {"tokens": self.size, "evictable_tokens": self.evictable_size, "snapshots": self.snapshots,
                "evictable_snapshots": self.state_evictable, "hits": self.hits, "misses": self.misses,
                "full_reprefills": self.full_reprefills}
