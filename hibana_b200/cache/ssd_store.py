"""Content-addressed object store of the SSD cache tier.

Objects are named by a hash chained over ALL tokens of the prefix they end, starting from a root hash of the
serving identity (model, revision, weight format, KV bytes per token, state bytes per slot, TP rank / size, ...):
another build, another rank or another model never matches, and one shared prefix is stored once. A file is
  header (magic, format, kind, key, payload sizes, CRC32 of the header) | payload segments | CRC32 of the payload
written as `<key>.tmp`, fdatasync'ed and renamed, so a crash leaves either the old state or a complete object; any
mismatch on read (magic, key, sizes, either CRC) is a miss, never an error. Writer threads (keyed by key hash, so
one object is only ever written by one thread) take O_DIRECT where the filesystem offers it. `flush` is O(1): it
bumps an epoch that is part of the root hash. Budget: least-recently-used objects are dropped when the stored
bytes exceed it. Reference: hibana/cache/ssd_store.py:72-97,104-160,269-396,439-553, docs/cache_design.md:193-252.
"""
from __future__ import annotations

import hashlib
import os
import queue
import struct
import threading
import zlib
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Optional, Sequence

MAGIC = b"HBNSSD1\n"
FORMAT = 1
KIND_KV, KIND_TAIL = 1, 2
BLOCK_TOKENS = 256
_HDR = struct.Struct("<8sIIQQQ32s")      # magic, format, kind, tokens, seg0 bytes, seg1 bytes, key
ALIGN = 4096


def root_hash(identity: dict, epoch: int = 0) -> bytes:
    h = hashlib.blake2b(digest_size=32)
    for k in sorted(identity):
        h.update(f"{k}={identity[k]};".encode())
    h.update(f"epoch={epoch}".encode())
    return h.digest()


def chain_hash(parent: bytes, tokens: Sequence[int], kind: int = KIND_KV) -> bytes:
    h = hashlib.blake2b(digest_size=32)
    h.update(parent)
    h.update(struct.pack("<I", kind))
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    return h.digest()


@dataclass
class Header:
    kind: int
    tokens: int
    seg0: int
    seg1: int
    key: bytes

    def pack(self) -> bytes:
        body = _HDR.pack(MAGIC, FORMAT, self.kind, self.tokens, self.seg0, self.seg1, self.key)
        return body + struct.pack("<I", zlib.crc32(body))

    @classmethod
    def unpack(cls, raw: bytes) -> Optional["Header"]:
        if len(raw) < _HDR.size + 4:
            return None
        body, (crc,) = raw[:_HDR.size], struct.unpack("<I", raw[_HDR.size:_HDR.size + 4])
        if zlib.crc32(body) != crc:
            return None
        magic, fmt, kind, tokens, s0, s1, key = _HDR.unpack(body)
        if magic != MAGIC or fmt != FORMAT:
            return None
        return cls(kind, tokens, s0, s1, key)


HEADER_BYTES = _HDR.size + 4


class SsdStore:
    def __init__(self, directory: str | os.PathLike, identity: dict, *, budget_bytes: int = 200 << 30,
                 writers: int = 4, direct: bool = True):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.identity = dict(identity)
        self.budget = budget_bytes
        self.direct = direct
        self.epoch = self._load_epoch()
        self.root = root_hash(self.identity, self.epoch)
        self._lock = threading.Lock()
        self._index: dict[bytes, int] = {}          # key -> bytes on disk
        self._lru: dict[bytes, int] = {}            # key -> logical tick
        self._tick = 0
        self.stored_bytes = 0
        self.writes = self.reads = self.misses = self.corrupt = self.dropped = 0
        self.write_gbs = 0.0            # measured rate of one writer (exponential average), for the tier's cost model
        self._tls = threading.local()
        self._queues = [queue.Queue() for _ in range(max(1, writers))]
        self._done: "queue.Queue[tuple[bytes, bool, object]]" = queue.Queue()
        self._threads = [threading.Thread(target=self._writer, args=(q,), daemon=True, name=f"ssd-writer-{i}")
                         for i, q in enumerate(self._queues)]
        for th in self._threads:
            th.start()
        self.scan()

    # ---- epochs (O(1) flush)
    def _epoch_file(self) -> Path:
        return self.dir / "EPOCH"

    def _load_epoch(self) -> int:
        try:
            return int(self._epoch_file().read_text().strip())
        except (OSError, ValueError):
            return 0

    def flush(self) -> None:
        """Forgets everything: new keys derive from a new root; old files are unlinked lazily by `scan`."""
        with self._lock:
            self.epoch += 1
            tmp = self._epoch_file().with_suffix(".tmp")
            tmp.write_text(str(self.epoch))
            os.replace(tmp, self._epoch_file())
            self.root = root_hash(self.identity, self.epoch)
            stale = list(self._index)
            self._index.clear()
            self._lru.clear()
            self.stored_bytes = 0
        for key in stale:
            self._unlink(key)

    # ---- paths
    def _path(self, key: bytes) -> Path:
        hx = key.hex()
        return self.dir / hx[:2] / f"{hx}.obj"

    def _unlink(self, key: bytes) -> None:
        try:
            self._path(key).unlink()
        except OSError:
            pass

    def scan(self) -> int:
        """Indexes complete objects of the current epoch left by an earlier process; removes temp files and
        objects whose header does not verify. Returns the number of objects kept."""
        kept = 0
        for sub in self.dir.iterdir():
            if not sub.is_dir():
                continue
            for f in sub.iterdir():
                if f.suffix == ".tmp":
                    f.unlink(missing_ok=True)
                    continue
                if f.suffix != ".obj":
                    continue
                try:
                    with open(f, "rb") as fh:
                        hdr = Header.unpack(fh.read(HEADER_BYTES))
                    size = f.stat().st_size
                except OSError:
                    hdr = None
                if hdr is None or hdr.key.hex() != f.stem:
                    f.unlink(missing_ok=True)
                    continue
                with self._lock:
                    if hdr.key not in self._index:
                        self._index[hdr.key] = size
                        self._tick += 1
                        self._lru[hdr.key] = self._tick
                        self.stored_bytes += size
                        kept += 1
        return kept

    # ---- index
    def contains(self, key: bytes) -> bool:
        with self._lock:
            return key in self._index

    def touch(self, key: bytes) -> None:
        with self._lock:
            if key in self._index:
                self._tick += 1
                self._lru[key] = self._tick

    def _enforce_budget(self) -> None:
        victims = []
        with self._lock:
            while self.stored_bytes > self.budget and self._lru:
                key = min(self._lru, key=self._lru.get)
                self.stored_bytes -= self._index.pop(key)
                del self._lru[key]
                victims.append(key)
                self.dropped += 1
        for key in victims:
            self._unlink(key)

    # ---- write path
    def write_async(self, key: bytes, kind: int, tokens: int, seg0: bytes | memoryview, seg1: bytes | memoryview = b"",
                    token: object = None, ready=None) -> None:
        """Queues an object; completion (key, ok, token) appears in `completions()`. The segments must stay
        untouched until then. `ready` (optional callable) is run by the writer thread before it touches the
        segments: a CUDA event's `synchronize`, so the engine thread never waits for the gather that fills them."""
        q = self._queues[int.from_bytes(key[:4], "little") % len(self._queues)]
        q.put((key, kind, tokens, seg0, seg1, token, ready))

    def completions(self) -> list:
        out = []
        while True:
            try:
                out.append(self._done.get_nowait())
            except queue.Empty:
                return out

    def drain(self, timeout: float = 30.0) -> None:
        for q in self._queues:
            q.join()

    def _writer(self, q: "queue.Queue") -> None:
        while True:
            item = q.get()
            try:
                if item is None:
                    return
                key, kind, tokens, seg0, seg1, token, ready = item
                if ready is not None:
                    ready()
                ok = self._write(key, kind, tokens, seg0, seg1)
                self._done.put((key, ok, token))
            finally:
                q.task_done()

    def _write(self, key: bytes, kind: int, tokens: int, seg0, seg1) -> bool:
        import time
        path = self._path(key)
        tmp = path.with_suffix(".tmp")
        hdr = Header(kind, tokens, len(seg0), len(seg1), key).pack()
        crc = zlib.crc32(seg1, zlib.crc32(seg0))
        parts = [hdr, seg0, seg1, struct.pack("<I", crc)]
        total = sum(len(p) for p in parts)
        t0 = time.perf_counter()
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            self._write_file(tmp, parts, total)
            os.replace(tmp, path)
        except OSError:
            try:
                tmp.unlink()
            except OSError:
                pass
            return False
        took = time.perf_counter() - t0
        with self._lock:
            self.stored_bytes += total - self._index.get(key, 0)
            self._index[key] = total
            self._tick += 1
            self._lru[key] = self._tick
            self.writes += 1
            if took > 0 and total >= (64 << 10):     # what one writer sustains, fdatasync included
                rate = total / took / 1e9
                self.write_gbs = rate if self.write_gbs == 0 else 0.8 * self.write_gbs + 0.2 * rate
        self._enforce_budget()
        return True

    def _bounce(self, nbytes: int):
        """This writer thread's page-aligned bounce buffer (grown on demand, reused across writes)."""
        import mmap
        buf = getattr(self._tls, "bounce", None)
        if buf is None or len(buf) < nbytes:
            if buf is not None:
                buf.close()
            buf = mmap.mmap(-1, max(nbytes, ALIGN))
            self._tls.bounce = buf
        return buf

    def _write_file(self, tmp: Path, parts: list, total: int) -> None:
        """O_DIRECT through an aligned bounce buffer where possible (the tail is padded and the file truncated to
        its true length afterwards), one gathered write otherwise; fdatasync before the rename either way. The
        segments are never joined in Python: the copy into the bounce buffer is a `memmove` outside the
        interpreter lock, so a writer thread does not hold up the engine thread for the length of a block."""
        import ctypes
        import numpy as np
        flags = os.O_WRONLY | os.O_CREAT | os.O_TRUNC
        fd = -1
        if self.direct and hasattr(os, "O_DIRECT"):
            try:
                fd = os.open(tmp, flags | os.O_DIRECT, 0o644)
            except OSError:
                fd = -1
        if fd >= 0:
            try:
                padded = (total + ALIGN - 1) // ALIGN * ALIGN
                buf = self._bounce(padded)
                base = ctypes.addressof(ctypes.c_char.from_buffer(buf))
                off = 0
                for p in parts:
                    if len(p):
                        src = np.frombuffer(p, dtype=np.uint8)
                        ctypes.memmove(base + off, src.ctypes.data, len(p))
                        off += len(p)
                if padded > total:
                    ctypes.memset(base + total, 0, padded - total)
                view = memoryview(buf)[:padded]
                try:
                    off = 0
                    while off < padded:
                        off += os.write(fd, view[off:min(off + (16 << 20), padded)])
                finally:
                    view.release()
                os.ftruncate(fd, total)
                os.fdatasync(fd)
                return
            except OSError:
                pass                                     # filesystem without O_DIRECT support for this file
            finally:
                os.close(fd)
        fd = os.open(tmp, flags, 0o644)
        try:
            views = [memoryview(p).cast("B") for p in parts if len(p)]
            while views:
                n = os.writev(fd, views[:16])
                while n and views:
                    if n >= len(views[0]):
                        n -= len(views[0])
                        views.pop(0)
                    else:
                        views[0] = views[0][n:]
                        n = 0
            os.fdatasync(fd)
        finally:
            os.close(fd)

    # ---- read path
    def read(self, key: bytes, kind: int) -> Optional[tuple[Header, bytes, bytes]]:
        """(header, seg0, seg1) or None on any damage (the damaged file is removed)."""
        with self._lock:
            known = key in self._index
        if not known:
            self.misses += 1
            return None
        path = self._path(key)
        try:
            raw = path.read_bytes()
        except OSError:
            raw = b""
        hdr = Header.unpack(raw[:HEADER_BYTES])
        good = (hdr is not None and hdr.key == key and hdr.kind == kind
                and len(raw) == HEADER_BYTES + hdr.seg0 + hdr.seg1 + 4)
        if good:
            seg0 = raw[HEADER_BYTES:HEADER_BYTES + hdr.seg0]
            seg1 = raw[HEADER_BYTES + hdr.seg0:HEADER_BYTES + hdr.seg0 + hdr.seg1]
            (crc,) = struct.unpack("<I", raw[-4:])
            good = zlib.crc32(seg1, zlib.crc32(seg0)) == crc
        if not good:
            self.corrupt += 1
            with self._lock:
                self.stored_bytes -= self._index.pop(key, 0)
                self._lru.pop(key, None)
            self._unlink(key)
            return None
        self.touch(key)
        self.reads += 1
        return hdr, seg0, seg1

    def read_into(self, key: bytes, kind: int, dst: memoryview) -> Optional[Header]:
        """Reads segment 0 of the object into `dst` (e.g. a pinned staging buffer); None on any damage."""
        got = self.read(key, kind)
        if got is None or len(got[1]) > len(dst):
            return None
        dst[:len(got[1])] = got[1]
        return got[0]

    def close(self) -> None:
        for q in self._queues:
            q.put(None)
        for th in self._threads:
            th.join(5)

    def stats(self) -> dict:
        with self._lock:
            return {"objects": len(self._index), "bytes": self.stored_bytes, "writes": self.writes,
                    "reads": self.reads, "misses": self.misses, "corrupt": self.corrupt, "dropped": self.dropped,
                    "epoch": self.epoch}
