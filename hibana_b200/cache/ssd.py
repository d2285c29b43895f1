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


class SsdTier:
    def __init__(self, store: SsdStore, kv_pool, *, min_prefix: int = MIN_PREFIX, min_gain: int = MIN_GAIN,
                 staging_blocks: int = 32, agree: Optional[Callable[[int], int]] = None):
        self.store, self.kv = store, kv_pool
        self.min_prefix, self.min_gain = min_prefix, min_gain
        self.agree = agree or (lambda n: n)
        self.token_bytes = kv_pool.bytes_per_token
        pin = kv_pool.device.type == "cuda"
        self.staging = Staging(staging_blocks, BLOCK_TOKENS * self.token_bytes, pin)
        self.backed_up = self.restored_tokens = self.skipped = 0

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
            if dev.type == "cuda":
                torch.cuda.current_stream(dev).synchronize()
            self.store.write_async(key, KIND_KV, BLOCK_TOKENS, memoryview(buf.numpy()), b"", token=i)
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
        """Engine-thread poll: returns staging buffers of finished writes. Returns the number completed."""
        done = self.store.completions()
        for _key, _ok, token in done:
            if token is not None:
                self.staging.give(token)
        return len(done)

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
        return n if n - have >= self.min_gain else 0

    def restore(self, tokens: Sequence[int], start: int, end: int, slots: Sequence[int]) -> int:
        """Reads blocks covering positions [start, end) (block aligned) into `slots` (one per position). Returns
        the first position NOT restored (== end on success; earlier when a block is damaged on any rank)."""
        assert start % BLOCK_TOKENS == 0 and end % BLOCK_TOKENS == 0 and len(slots) == end - start
        keys = self._block_keys(tokens, end // BLOCK_TOKENS)
        dev = self.kv.device
        good = start
        i = self.staging.take()
        if i is None:
            return self.agree(start)
        buf = self.staging.bufs[i]
        try:
            for b in range(start // BLOCK_TOKENS, end // BLOCK_TOKENS):
                hdr = self.store.read_into(keys[b], KIND_KV, memoryview(buf.numpy()))
                if hdr is None or hdr.tokens != BLOCK_TOKENS or hdr.seg0 != BLOCK_TOKENS * self.token_bytes:
                    break
                lo = b * BLOCK_TOKENS - start
                ids = torch.tensor(slots[lo:lo + BLOCK_TOKENS], dtype=torch.int32, device=dev)
                self.kv.copy_payload(ids, buf, to_pool=True)
                if dev.type == "cuda":
                    torch.cuda.current_stream(dev).synchronize()     # the buffer is reused for the next block
                good = (b + 1) * BLOCK_TOKENS
        finally:
            self.staging.give(i)
        good = self.agree(good)
        self.restored_tokens += max(good - start, 0)
        return good

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

    def stats(self) -> dict:
        return {"backed_up_blocks": self.backed_up, "restored_tokens": self.restored_tokens, "skipped": self.skipped,
                **self.store.stats()}
