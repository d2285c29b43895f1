"""StateManager: the only component that moves KV-slot / state-slot ownership or advances `committed_len`.

Ownership model: positions [0, shared_len) of a request's `kv_slots` belong to the radix tree (the request holds
one TreeLock at the node ending at shared_len); positions from shared_len on are private. After every prefill
chunk and at release the committed prefix is inserted into the tree, which adopts the private slots and moves the
lock deeper. Speculative steps are a transaction: reserve -> (verify) -> commit(count) / rollback.
Reference: hibana/cache/request_state.py:62-475 and docs/interfaces.md:38-93.
"""
from __future__ import annotations

from typing import Optional, Sequence

from .kv_pool import KvPool
from .radix import RadixCache, Snapshot
from .state_pool import StatePool


class StateManager:
    def __init__(self, kv: KvPool, state_pool: Optional[StatePool] = None, *, cache: bool = True,
                 decode_reserve: int = 64):
        self.kv, self.states = kv, state_pool
        self.decode_reserve = decode_reserve
        self.cache: Optional[RadixCache] = None
        if cache:
            self.cache = RadixCache(kv.free, state_pool.free if state_pool is not None else None,
                                    needs_state=state_pool is not None)
        self.live: dict[int, object] = {}      # rid -> request (for invariants)
        self.poisoned = False

    # ---- admission
    def _budget(self, req) -> tuple[int, int]:
        """(tokens needed, tokens obtainable) without changing anything."""
        tokens = req.all_ids[:-1] if req.output_ids else req.prompt_ids
        matched = 0
        if self.cache is not None and req.cacheable:
            m = self.cache.match(tokens[:max(len(tokens) - 1, 0)], split=False)
            matched = m.state_length if self.cache.needs_state else m.length
        need = len(tokens) - matched + min(self.decode_reserve, max(req.remaining, 1))
        have = self.kv.free_count + (self.cache.evictable_size if self.cache is not None else 0)
        return need, have

    def can_admit(self, req, promised: int = 0) -> bool:
        """Pure: budgets the uncached suffix plus a decode reserve against free + evictable memory, less `promised`
        slots: what requests admitted earlier have yet to take for the rest of their prompts (without that term a
        burst of long prompts is admitted together, none can finish its prefill, and retraction and re-admission
        chase each other)."""
        need, have = self._budget(req)
        if need > have - promised:
            return False
        if self.states is not None:
            spare = self.states.free_count + (self.cache.state_evictable if self.cache is not None else 0)
            if spare < 2:
                return False
        return True

    def admit(self, req) -> None:
        """Matches the prompt against the cache, locks the usable prefix, takes a state slot and copies the
        matched snapshot into it. On failure everything taken is returned."""
        tokens = req.all_ids[:-1] if req.output_ids else req.prompt_ids
        req.kv_slots, req.cached_len, req.shared_len, req.lock = [], 0, 0, None
        req.branch_at = 0
        try:
            if self.cache is not None and req.cacheable:
                # never match the whole prompt: the last token must be run to produce logits
                m = self.cache.match(tokens[:max(len(tokens) - 1, 0)])
                node, length = self.cache.usable(m)
                req.branch_at = m.length if length < m.length else 0
                req.lock = self.cache.lock(node)
                if length:
                    req.kv_slots = node.path_slots()[:length]
                    req.cached_len = req.shared_len = length
            if self.states is not None:
                req.state_slot = self._alloc_state()
                snap = req.lock.node.snapshot if (req.lock is not None and req.cached_len) else None
                if snap is not None:
                    self.states.copy_slot(snap.slot, req.state_slot)
                else:
                    self.states.zero_slot(req.state_slot)
        except Exception:
            self._drop(req)
            raise
        req.committed_len = req.cached_len
        self.live[req.rid] = req

    def begin_ssd_restore(self, tokens: Sequence[int], tier):
        """Before admission: when the SSD tier holds at least `tier.min_gain` more tokens of this prompt than the
        GPU cache, allocates slots and starts reading the blocks into them (`SsdTier.restore_async`). Returns the
        job, or None when a restore is not worth it. KV-only models (a recurrent model also needs the state
        snapshot of the tail object; without one the restored KV could not be resumed from)."""
        if self.cache is None or self.states is not None or tier is None:
            return None
        tokens = list(tokens[:max(len(tokens) - 1, 0)])
        m = self.cache.match(tokens, split=False)
        have = m.length
        n = tier.worth(tokens, have)
        if not n:
            return None
        m = self.cache.match(tokens[:have])            # split so that a node ends exactly at `have`
        lock = self.cache.lock(m.node)                  # the allocation below must not evict the matched path
        try:
            fresh = self._alloc_kv(n - have)
        except MemoryError:
            self.cache.unlock(lock)
            return None
        from .ssd_store import BLOCK_TOKENS
        start = have // BLOCK_TOKENS * BLOCK_TOKENS
        ids = [0] * (have - start) + fresh              # rows the tree already has land in the dummy slot
        job = tier.restore_async(tokens, start, n, ids)
        job.context = {"lock": lock, "fresh": fresh, "have": have, "node": m.node, "tokens": tokens, "n": n}
        return job

    def finish_ssd_restore(self, job, tier) -> int:
        """After the job finished: publishes the restored rows in the tree (the admission that follows simply
        hits), frees what did not come back, drops the path lock. Returns tokens restored."""
        c = job.context
        have, fresh, n = c["have"], c["fresh"], c["n"]
        try:
            good = max(tier.finish(job), have)
            if good < n:
                self.kv.free(fresh[good - have:])
                fresh = fresh[:good - have]
            if fresh:
                path = c["node"].path_slots()[:have]
                _node, adopted = self.cache.insert(c["tokens"][:good], path + fresh, start=have)
                if adopted < good:                      # someone cached the same tokens meanwhile
                    self.kv.free(fresh[adopted - have:])
            return max(good - have, 0)
        finally:
            self.cache.unlock(c["lock"])

    def restore_from_ssd(self, tokens: Sequence[int], tier) -> int:
        """Blocking form (offline tools, tests): begin, drive the job to the end, finish. Returns tokens restored."""
        import time
        job = self.begin_ssd_restore(tokens, tier)
        if job is None:
            return 0
        while not tier.pump(job):
            time.sleep(0.0005)
        return self.finish_ssd_restore(job, tier)

    def _alloc_state(self) -> int:
        if self.states.free_count == 0 and self.cache is not None:
            self.cache.evict_snapshots(1)
        return self.states.alloc()

    def _alloc_kv(self, n: int) -> list:
        short = n - self.kv.free_count
        if short > 0 and self.cache is not None:
            self.cache.evict(short)
        return self.kv.alloc(n)

    # ---- growth
    def extend(self, req, n: int) -> list:
        """Allocates KV slots for the next n positions of the request (evicting unlocked cache if needed)."""
        slots = self._alloc_kv(n)
        req.kv_slots.extend(slots)
        return slots

    def after_prefill(self, req, final: bool, snapshot_spare: Optional[bool] = None) -> None:
        """Publishes the committed prefix (KV, and a state snapshot at its end) after a prefill forward."""
        if self.cache is None or not req.cacheable or self.poisoned:
            return
        self._publish(req, req.committed_len, spare=(not final) if snapshot_spare is None else snapshot_spare)

    def _publish(self, req, length: int, spare: bool) -> None:
        if length <= req.shared_len:
            return
        tokens = req.all_ids[:length]
        node, adopted = self.cache.insert(tokens, req.kv_slots[:length], start=req.shared_len)
        if adopted == req.shared_len and self.states is not None:
            # The tree already holds these tokens (cached KV without a usable snapshot made this request re-run
            # them): keep the private copy, but leave a snapshot on the existing path so the next request resumes.
            m = self.cache.match(tokens)
            if m.length == length and m.node.snapshot is None and m.node is not self.cache.root:
                try:
                    slot = self._alloc_state()
                except MemoryError:
                    return
                self.states.copy_slot(req.state_slot, slot)
                self.cache.set_snapshot(m.node, Snapshot(slot, length, spare=spare))
            return
        if adopted > req.shared_len:
            req.lock = self.cache.move_lock(req.lock, node) if req.lock is not None else self.cache.lock(node)
            req.shared_len = adopted
            if self.states is not None and adopted == length and node.snapshot is None:
                try:
                    slot = self._alloc_state()
                except MemoryError:
                    return     # nothing waits for a slot: the prefix stays resumable only at earlier snapshots
                self.states.copy_slot(req.state_slot, slot)
                old = self.cache.set_snapshot(node, Snapshot(slot, length, spare=spare))
                if old is not None:
                    self.states.free(old.slot)

    # ---- speculative transaction
    def reserve(self, reqs: Sequence, width: int) -> list[list]:
        """Slots for `width` candidate positions of every request; all or nothing."""
        taken = []
        try:
            for r in reqs:
                slots = self._alloc_kv(width)
                r.kv_slots.extend(slots)
                r.reserved = width
                taken.append(slots)
        except MemoryError:
            for r, slots in zip(reqs, taken):
                del r.kv_slots[len(r.kv_slots) - len(slots):]
                self.kv.free(slots)
                r.reserved = 0
            raise
        return taken

    def commit(self, req, count: int) -> None:
        """Keeps exactly `count` of the reserved positions; frees the rest."""
        extra = req.reserved - count
        assert 0 <= count <= req.reserved
        if extra:
            drop = req.kv_slots[len(req.kv_slots) - extra:]
            del req.kv_slots[len(req.kv_slots) - extra:]
            self.kv.free(drop)
        req.reserved = 0
        req.committed_len = len(req.kv_slots)

    def rollback(self, req) -> None:
        """Frees the pending positions and disables caching (in-place recurrent writes are not undone)."""
        if req.reserved:
            drop = req.kv_slots[len(req.kv_slots) - req.reserved:]
            del req.kv_slots[len(req.kv_slots) - req.reserved:]
            self.kv.free(drop)
            req.reserved = 0
        req.cacheable = False

    def poison(self) -> None:
        """After a failed forward nothing of the batch may be cached or retried."""
        self.poisoned = True
        for r in self.live.values():
            r.cacheable = False

    # ---- release
    def _drop(self, req) -> None:
        private = req.kv_slots[req.shared_len:] if hasattr(req, "shared_len") else req.kv_slots
        if private:
            self.kv.free(private)
        req.kv_slots = []
        if self.cache is not None and req.lock is not None:
            self.cache.unlock(req.lock)
        req.lock = None
        if self.states is not None and req.state_slot:
            self.states.free(req.state_slot)
            req.state_slot = 0
        req.shared_len = req.cached_len = 0
        self.live.pop(req.rid, None)

    def release(self, req) -> None:
        """Idempotent. Transfers the valid prefix (prompt + all but the pending token) into the cache, with the
        request's own state slot as the reply-end snapshot, then frees what is left."""
        if req.rid not in self.live:
            return
        if self.cache is not None and req.cacheable and not self.poisoned and req.reserved == 0:
            valid = min(req.committed_len, len(req.kv_slots), max(req.total_len - 1, 0))
            if valid > req.shared_len:
                self._publish(req, valid, spare=True)
        self._drop(req)

    def retract(self, req) -> None:
        self._drop(req)
        req.committed_len = 0

    # ---- invariants
    def check(self) -> None:
        self.kv.check()
        tree = self.cache.all_slots() if self.cache is not None else []
        private = []
        for r in self.live.values():
            assert len(r.kv_slots) >= r.shared_len
            private.extend(r.kv_slots[r.shared_len:])
        owned = tree + private
        assert len(set(owned)) == len(owned), "a KV slot has two owners"
        assert len(owned) + self.kv.free_count == self.kv.slots, (len(owned), self.kv.free_count, self.kv.slots)
        if self.cache is not None:
            self.cache.check()
            locks = sum(1 for r in self.live.values() if r.lock is not None)
            assert sum(c.lock_ref for c in self.cache.root.children.values()) <= locks
        if self.states is not None:
            self.states.check()
            held = [r.state_slot for r in self.live.values() if r.state_slot]
            snaps = self.cache.snapshots if self.cache is not None else 0
            assert len(held) + snaps + self.states.reserved + self.states.free_count == self.states.slots

    def stats(self) -> dict:
        out = {"kv_free": self.kv.free_count, "kv_slots": self.kv.slots, "live_requests": len(self.live)}
        if self.cache is not None:
            out.update(self.cache.stats())
        if self.states is not None:
            out["state_free"] = self.states.free_count
        return out
