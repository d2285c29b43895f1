"""Per-layer-embedding ("PLE") n-gram table: a table of small rows (160 bytes) far larger than GPU memory, sharded
over files on NVMe; every token needs a few rows (hashes of its trailing n-grams). `PleTable.gather` fetches a
batch of rows into pinned host memory with the C++ gatherer (csrc/row_gather.cpp: page-cache pass on the calling
thread, then a thread pool of blocking reads) and moves them to the device in one async copy. A table small enough to
live in GPU memory is served by a device-resident copy and a plain index_select instead.
Reference: hibana/model/flashnext/ple.py:34-42,173-202, hibana/kernels/csrc/ple_gather.cpp.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch

from .. import _native as nv

_LIB = None


def _host_lib():
    """The row gatherer needs no GPU: load the shared library even where no CUDA device exists."""
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(str(nv.LIB_PATH))
        lib.hb_rows_open.restype = ctypes.c_void_p
        lib.hb_rows_open.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
        lib.hb_rows_add_shard.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        lib.hb_rows_gather.restype = ctypes.c_longlong
        lib.hb_rows_gather.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                       ctypes.c_void_p]
        lib.hb_rows_close.argtypes = [ctypes.c_void_p]
        _LIB = lib
    return _LIB


def ngram_rows(token_ids: Sequence[int], orders: Sequence[int], table_rows: int, rows_per_order: int = 1) -> np.ndarray:
    """Row ids for every token: one row per n-gram order (hash of the last n tokens, FNV-1a folded to the table)."""
    ids = np.asarray(token_ids, dtype=np.int64)
    out = np.empty((len(ids), len(orders) * rows_per_order), dtype=np.int64)
    for oi, n in enumerate(orders):
        h = np.full(len(ids), 0xCBF29CE484222325, dtype=np.uint64)
        for back in range(n):
            shifted = np.concatenate((np.zeros(min(back, len(ids)), dtype=np.int64), ids[:max(len(ids) - back, 0)]))
            h = (h ^ shifted.astype(np.uint64)) * np.uint64(0x100000001B3)
        for j in range(rows_per_order):
            out[:, oi * rows_per_order + j] = ((h >> np.uint64(7 * j)) % np.uint64(table_rows)).astype(np.int64)
    return out


class PleTable:
    def __init__(self, shard_paths: Sequence[str | os.PathLike], row_bytes: int, rows_per_shard: int,
                 device="cpu", threads: int = 8, resident_limit_bytes: int = 0):
        self.row_bytes, self.rows_per_shard = row_bytes, rows_per_shard
        self.rows = rows_per_shard * len(shard_paths)
        self.device = torch.device(device)
        self.cold_rows = 0
        self._resident: Optional[torch.Tensor] = None
        total = self.rows * row_bytes
        if resident_limit_bytes and total <= resident_limit_bytes:
            parts = [torch.from_numpy(np.fromfile(p, dtype=np.uint8)) for p in shard_paths]
            self._resident = torch.cat(parts).view(self.rows, row_bytes).to(self.device)
            self._h = None
            return
        lib = _host_lib()
        self._h = lib.hb_rows_open(row_bytes, rows_per_shard, threads)
        if not self._h:
            raise ValueError("bad table geometry")
        for p in shard_paths:
            if lib.hb_rows_add_shard(self._h, str(Path(p)).encode()) != 0:
                raise FileNotFoundError(p)

    def gather(self, rows: np.ndarray | torch.Tensor) -> torch.Tensor:
        """rows: int64 [..] -> uint8 [.., row_bytes] on the table's device."""
        if self._resident is not None:
            idx = torch.as_tensor(np.asarray(rows) if not isinstance(rows, torch.Tensor) else rows).to(self.device)
            return self._resident.index_select(0, idx.reshape(-1).long()).view(*idx.shape, self.row_bytes)
        r = np.ascontiguousarray(np.asarray(rows.cpu() if isinstance(rows, torch.Tensor) else rows), dtype=np.int64)
        n = r.size
        host = torch.empty(n, self.row_bytes, dtype=torch.uint8, pin_memory=self.device.type == "cuda")
        cold = ctypes.c_longlong(0)
        got = _host_lib().hb_rows_gather(self._h, r.ctypes.data, n, host.data_ptr(), ctypes.byref(cold))
        if got != n:
            raise IOError(f"row gather failed at row index {-got - 1 if got < 0 else got}")
        self.cold_rows += int(cold.value)
        return host.to(self.device, non_blocking=True).view(*r.shape, self.row_bytes)

    def close(self) -> None:
        if getattr(self, "_h", None):
            _host_lib().hb_rows_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
