"""SSD tier of the prefix cache: KV rows (and recurrent-state snapshots) of long prefixes survive eviction and
restarts on NVMe and come back with one gather / scatter kernel per direction.

Objects (cache/ssd_store.py): `.kv` blocks of 256 tokens holding every layer's K and V rows of the block back to
back, and a `.tail` per backed-up prefix with the partial last block, the recurrent-state snapshot at the prefix end
and an opaque drafter payload. Keys chain over all tokens, so a shared prefix is stored once and blocks are found
by walking the chain. Rules kept from the reference: prefixes shorter than `min_prefix` tokens are not backed up; a
restore must gain at least `min_gain` tokens over what the GPU cache already holds; nothing ever waits for the
tier (no free staging buffer -> the backup is skipped); with tensor parallelism each rank stores its own heads and
a restore proceeds only as far as EVERY rank read intact (`agree` = min over ranks).
Data path: KvPool.copy_payload gathers the rows of a block from all layers straight into a pinned host buffer
(the kernel writes over PCIe; csrc/kv_copy.cu), a writer thread streams that buffer to the file; restores read into
a pinned buffer and scatter it into freshly allocated slots.
Reference: hibana/cache/ssd.py:96-101,131-246,413-643,764-871,946-1250, docs/cache_design.md:193-306.
"""
from __future__ import annotations

import time

from concurrent.futures import Future, ThreadPoolExecutor
from typing import Callable, Optional, Sequence

import torch

from .ssd_store import BLOCK_TOKENS, KIND_KV, KIND_TAIL, SsdStore, chain_hash

MIN_PREFIX = 4096
MIN_GAIN = 2048


class Staging:
    """A few pinned host buffers, one block each. `take` never blocks."""

    def __init__(self, count: int, nbytes: int, pin: bool):
        self.nbytes = nbytes
        self.bufs = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=pin) for _ in range(count)]
        self.free = list(range(count))

    def take(self) -> Optional[int]:
        return self.free.pop() if self.free else None

    def give(self, i: int) -> None:
        self.free.append(i)


class RestoreJob:
    """One prefix coming back from disk: blocks [start, end) of `tokens` into `slots`. Reader threads fill staging
    buffers ahead of the engine thread, which scatters finished blocks in order (`SsdTier.pump`) without ever
    waiting for a read or for the GPU."""

    def __init__(self, tokens: Sequence[int], start: int, end: int, slots: Sequence[int], keys: list):
        self.tokens, self.start, self.end, self.slots, self.keys = tokens, start, end, list(slots), keys
        self.first, self.last = start // BLOCK_TOKENS, end // BLOCK_TOKENS
        self.next_read = self.next_scatter = self.first
        self.reads: dict[int, tuple[int, Future]] = {}      # block -> (staging buffer, pending read)
        self.good = start                                   # first position not yet scattered
        self.failed = False
        self.t0 = time.perf_counter()
        self.context: dict = {}                             # owner's bookkeeping (locks, fresh slots)

    @property
    def finished(self) -> bool:
        return self.failed or self.next_scatter >= self.last


class SsdTier:
    def __init__(self, store: SsdStore, kv_pool, *, min_prefix: int = MIN_PREFIX, min_gain: int = MIN_GAIN,
                 staging_blocks: int = 32, agree: Optional[Callable[[int], int]] = None, readers: int = 4,
                 read_ahead: int = 8):
        self.store, self.kv = store, kv_pool
        self.min_prefix, self.min_gain = min_prefix, min_gain
        self.agree = agree or (lambda n: n)
        self.token_bytes = kv_pool.bytes_per_token
        pin = kv_pool.device.type == "cuda"
        self.staging = Staging(staging_blocks, BLOCK_TOKENS * self.token_bytes, pin)
        self.backed_up = self.restored_tokens = self.skipped = 0
        self.readers = ThreadPoolExecutor(max_workers=readers, thread_name_prefix="hibana-ssd-read")
        self.read_ahead = read_ahead
        self._scattered: list = []       # (CUDA event or None, staging buffer) of scatters still in flight
        self.trace = None                # optional callable(event: str, **fields) (engine/traces.py)
        # Cost model: a restore pays only when reading a token's KV back is faster than computing it again. On this
        # class of GPU a prefill chunk runs at tens of thousands of tokens per second while a token of bf16 KV of a
        # 27B model is 256 KiB, so whether the tier pays depends on the KV format and the disk. Both rates are
        # measured while serving (exponential averages); `prefill_tok_s` is fed by the executor. 0 = not known yet:
        # the tier is then used whenever the prefix policy allows it.
        self.read_gbs = 0.0
        self.prefill_tok_s = 0.0
        self.declined = 0

    def note_read(self, nbytes: int, seconds: float) -> None:
        if seconds > 0 and nbytes > 0:
            rate = nbytes / seconds / 1e9
            self.read_gbs = rate if self.read_gbs == 0 else 0.8 * self.read_gbs + 0.2 * rate

    def note_prefill(self, tokens: int, seconds: float) -> None:
        if seconds > 0 and tokens >= 256:
            rate = tokens / seconds
            self.prefill_tok_s = rate if self.prefill_tok_s == 0 else 0.8 * self.prefill_tok_s + 0.2 * rate

    def disk_gbs(self) -> float:
        """The rate a restore can expect: measured reads, else what the writers sustained (a disk that takes a
        block slowly will not give it back fast), else 0 = not known."""
        if self.read_gbs > 0:
            return self.read_gbs
        return getattr(self.store, "write_gbs", 0.0) * max(len(getattr(self.store, "_queues", ())), 1)

    def pays(self, tokens: int) -> bool:
        """True when bringing `tokens` tokens back from disk is expected to beat prefilling them again. Backups ask
        the same question (`on_evict`): a block nobody would read back is not worth writing."""
        rate = self.disk_gbs()
        if rate <= 0 or self.prefill_tok_s <= 0 or tokens <= 0:
            return True
        restore_s = tokens * self.token_bytes / (rate * 1e9)
        return restore_s < 0.8 * tokens / self.prefill_tok_s

    # ---- keys
    def _block_keys(self, tokens: Sequence[int], nblocks: int) -> list[bytes]:
        keys, prev = [], self.store.root
        for b in range(nblocks):
            prev = chain_hash(prev, tokens[b * BLOCK_TOKENS:(b + 1) * BLOCK_TOKENS], KIND_KV)
            keys.append(prev)
        return keys

    # ---- backup
    def backup(self, tokens: Sequence[int], slots: Sequence[int], state: Optional[bytes] = None,
               aux: bytes = b"") -> int:
        """Queues every block of the prefix that is not on disk yet, and its tail. Returns blocks queued."""
        n = min(len(tokens), len(slots))
        if n < self.min_prefix:
            return 0
        nblocks = n // BLOCK_TOKENS
        keys = self._block_keys(tokens, nblocks)
        dev = self.kv.device
        queued = 0
        for b, key in enumerate(keys):
            if self.store.contains(key):
                self.store.touch(key)
                continue
            i = self.staging.take()
            if i is None:
                self.skipped += 1
                break                      # nothing waits for the tier; later blocks would be unreachable anyway
            ids = torch.tensor(slots[b * BLOCK_TOKENS:(b + 1) * BLOCK_TOKENS], dtype=torch.int32, device=dev)
            buf = self.staging.bufs[i]
            self.kv.copy_payload(ids, buf, to_pool=False)
            ready = None
            if dev.type == "cuda":      # the writer thread waits for the gather; the engine thread moves on, and
                ev = torch.cuda.Event()  # the slots may be freed at once (later kernels queue behind the gather)
                ev.record(torch.cuda.current_stream(dev))
                ready = ev.synchronize
            self.store.write_async(key, KIND_KV, BLOCK_TOKENS, memoryview(buf.numpy()), b"", token=i, ready=ready)
            queued += 1
        else:
            # tail: the partial last block + the snapshot of the recurrent state at the end of the prefix
            rest = n - nblocks * BLOCK_TOKENS
            parent = keys[-1] if keys else self.store.root
            tkey = chain_hash(parent, tokens[nblocks * BLOCK_TOKENS:n], KIND_TAIL)
            if (rest or state is not None) and not self.store.contains(tkey):
                ids = torch.tensor(slots[nblocks * BLOCK_TOKENS:n], dtype=torch.int32, device=dev)
                pay = torch.empty(rest * self.token_bytes, dtype=torch.uint8, pin_memory=dev.type == "cuda")
                if rest:
                    self.kv.copy_payload(ids, pay, to_pool=False)
                    if dev.type == "cuda":
                        torch.cuda.current_stream(dev).synchronize()
                meta = len(state or b"").to_bytes(8, "little") + (state or b"") + aux
                self.store.write_async(tkey, KIND_TAIL, rest, bytes(pay.numpy()), meta, token=None)
        self.backed_up += queued
        return queued

    def step(self) -> int:
        """Engine-thread poll: returns staging buffers of finished writes and of scatters the GPU has completed.
        Returns the number of writes completed."""
        done = self.store.completions()
        for _key, _ok, token in done:
            if token is not None:
                self.staging.give(token)
        keep = []
        for ev, i in self._scattered:
            if ev is None or ev.query():
                self.staging.give(i)
            else:
                keep.append((ev, i))
        self._scattered = keep
        return len(done)

    # ---- asynchronous restore
    def restore_async(self, tokens: Sequence[int], start: int, end: int, slots: Sequence[int]) -> RestoreJob:
        """Starts bringing blocks [start, end) (block aligned) back into `slots`; drive it with `pump`."""
        assert start % BLOCK_TOKENS == 0 and end % BLOCK_TOKENS == 0 and len(slots) == end - start
        job = RestoreJob(tokens, start, end, slots, self._block_keys(tokens, end // BLOCK_TOKENS))
        self.pump(job)
        return job

    def _read_block(self, key: bytes, i: int):
        return self.store.read_into(key, KIND_KV, memoryview(self.staging.bufs[i].numpy()))

    def pump(self, job: RestoreJob) -> bool:
        """Engine-thread step of a restore: hands free staging buffers to the reader threads (up to `read_ahead`
        blocks ahead), scatters every block whose read has finished, in order, with one kernel each, and never
        blocks: an unfinished read or a busy buffer just means "call again". Returns job.finished."""
        self.step()
        while (not job.failed and job.next_read < job.last and len(job.reads) < self.read_ahead):
            i = self.staging.take()
            if i is None:
                break
            job.reads[job.next_read] = (i, self.readers.submit(self._read_block, job.keys[job.next_read], i))
            job.next_read += 1
        dev = self.kv.device
        while job.next_scatter < job.last and job.next_scatter in job.reads:
            i, fut = job.reads[job.next_scatter]
            if not fut.done():
                break
            del job.reads[job.next_scatter]
            hdr = fut.result()
            if (job.failed or hdr is None or hdr.tokens != BLOCK_TOKENS
                    or hdr.seg0 != BLOCK_TOKENS * self.token_bytes):
                job.failed = True            # damaged or missing: the prefix ends before this block
                self.staging.give(i)
                continue
            b = job.next_scatter
            lo = b * BLOCK_TOKENS - job.start
            ids = torch.tensor(job.slots[lo:lo + BLOCK_TOKENS], dtype=torch.int32)
            if dev.type == "cuda":
                ids = ids.pin_memory().to(dev, non_blocking=True)
            self.kv.copy_payload(ids, self.staging.bufs[i], to_pool=True)
            ev = None
            if dev.type == "cuda":
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(dev))
            self._scattered.append((ev, i))
            job.next_scatter += 1
            job.good = (b + 1) * BLOCK_TOKENS
        if job.failed:
            for b in list(job.reads):        # reads still in flight: give their buffers back once they return
                i, fut = job.reads[b]
                if fut.done():
                    del job.reads[b]
                    self.staging.give(i)
            if job.reads:
                return False
        if job.finished:
            took = time.perf_counter() - job.t0
            self.note_read(max(job.good - job.start, 0) * self.token_bytes, took)
            if self.trace is not None:
                self.trace("ssd_restore", start=job.start, end=job.end, good=job.good, failed=job.failed,
                           seconds=round(took, 4), read_gbs=round(self.read_gbs, 2))
        return job.finished

    def finish(self, job: RestoreJob) -> int:
        """After `pump` returned True: the first position NOT restored, agreed over the ranks."""
        good = self.agree(job.good)
        self.restored_tokens += max(good - job.start, 0)
        return good

    # ---- lookup / restore
    def match(self, tokens: Sequence[int]) -> int:
        """Tokens of `tokens` restorable from disk as whole blocks (the chain stops at the first missing one)."""
        nblocks = len(tokens) // BLOCK_TOKENS
        prev, n = self.store.root, 0
        for b in range(nblocks):
            prev = chain_hash(prev, tokens[b * BLOCK_TOKENS:(b + 1) * BLOCK_TOKENS], KIND_KV)
            if not self.store.contains(prev):
                break
            n += BLOCK_TOKENS
        return n

    def worth(self, tokens: Sequence[int], have: int) -> int:
        """Tokens a restore would bring back, or 0 when it gains less than `min_gain` over `have` cached ones."""
        n = self.agree(self.match(tokens))
        if n - have >= self.min_gain and not self.pays(n - have):
            self.declined += 1
            return 0
        return n if n - have >= self.min_gain else 0

    def restore(self, tokens: Sequence[int], start: int, end: int, slots: Sequence[int]) -> int:
        """Blocking form of `restore_async` (tests, tools): returns the first position NOT restored (== end on
        success; earlier when a block is damaged on any rank)."""
        import time
        job = self.restore_async(tokens, start, end, slots)
        while not self.pump(job):
            time.sleep(0.0005)
        if self.kv.device.type == "cuda":
            torch.cuda.current_stream(self.kv.device).synchronize()
        self.step()
        return self.finish(job)

    def read_tail(self, tokens: Sequence[int]) -> Optional[tuple[int, bytes, Optional[bytes], bytes]]:
        """(tail tokens, their KV payload, state snapshot or None, drafter payload) of the prefix `tokens`."""
        nblocks = len(tokens) // BLOCK_TOKENS
        keys = self._block_keys(tokens, nblocks)
        parent = keys[-1] if keys else self.store.root
        got = self.store.read(chain_hash(parent, tokens[nblocks * BLOCK_TOKENS:], KIND_TAIL), KIND_TAIL)
        if got is None:
            return None
        hdr, pay, meta = got
        slen = int.from_bytes(meta[:8], "little")
        state = meta[8:8 + slen] if slen else None
        return hdr.tokens, pay, state, meta[8 + slen:]

    # ---- eviction / shutdown
    def on_evict(self, node) -> None:
        """Radix-tree hook, called before the KV of an unlocked leaf is freed: the whole path down to the leaf is
        backed up first (blocks already on disk are skipped), so that an evicted long prefix comes back from NVMe
        instead of being prefilled again. Copies are queued on the stream; nothing here waits."""
        tokens, slots, n = [], [], node
        while n is not None and n.parent is not None:
            tokens[:0], slots[:0] = n.tokens, n.slots
            n = n.parent
        if not self.pays(len(tokens)):       # nobody would read it back: computing it again is faster
            self.declined += 1
            return
        if self.backup(tokens, slots):
            node.on_ssd = True

    def persist(self, cache) -> int:
        """Shutdown: backs up every cached path of at least `min_prefix` tokens and waits for the writers."""
        queued = 0
        for leaf in list(cache._leaves()):
            tokens, slots, n = [], [], leaf
            while n is not None and n.parent is not None:
                tokens[:0], slots[:0] = n.tokens, n.slots
                n = n.parent
            while True:
                got = self.backup(tokens, slots)
                queued += got
                if got == 0 or self.skipped == 0:
                    break
                self.store.drain()           # staging was exhausted: let the writers catch up, then continue
                self.step()
                self.skipped = 0
        self.store.drain()
        self.step()
        return queued

    def stats(self) -> dict:
        return {"backed_up_blocks": self.backed_up, "restored_tokens": self.restored_tokens, "skipped": self.skipped,
                "declined": self.declined, "read_gbs": round(self.read_gbs, 2),
                "write_gbs_per_writer": round(getattr(self.store, "write_gbs", 0.0), 2),
                "prefill_tok_s": round(self.prefill_tok_s), **self.store.stats()}
