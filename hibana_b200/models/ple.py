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


# --------------------------------------------------------------------------------------------- the model layer
ROW_DIM = 160        # fp8 values per table row (the reference's 160-byte rows)


def gemma_group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """RMS norm over each of `groups` equal slices of the last dim, weight (1 + w), bf16 result."""
    t = x.shape[0]
    xf = x.float().view(t, groups, -1)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float().view(groups, -1))
    return y.view(t, -1).to(torch.bfloat16)


def dilated_conv_ragged(x: torch.Tensor, weight: torch.Tensor, dilation: int, window: torch.Tensor,
                        slot_in: torch.Tensor, slot_out: torch.Tensor, q_indptr: Optional[torch.Tensor],
                        has_init: Optional[torch.Tensor]) -> torch.Tensor:
    """Depth-wise causal convolution over time with a dilation, continuing every sequence's window.

    x [T, C] rows of B sequences (row ranges `q_indptr`, or one row each), weight [C, K] (tap K - 1 is the current
    row), window [slots, C, S] with S = (K - 1) * dilation: the S rows before the sequence's next row, newest last.
    Reads the windows at `slot_in`, writes the windows after the rows at `slot_out`, returns [T, C] in x's dtype.
    Everything is index arithmetic on the device (no host read), so the call can sit inside a CUDA graph.
    """
    t, c = x.shape
    k = weight.shape[1]
    s = (k - 1) * dilation
    dev = x.device
    b = slot_in.shape[0]
    rows = torch.arange(t, device=dev)
    if q_indptr is None:
        seq, local, start = rows, torch.zeros_like(rows), rows
        length = torch.ones(b, dtype=torch.int64, device=dev)
    else:
        ip = q_indptr.long()
        seq = torch.bucketize(rows, ip[1:], right=True).clamp_(max=b - 1)
        start = ip[:-1][seq]
        local = rows - start
        length = ip[1:] - ip[:-1]
    prev = window.index_select(0, slot_in.long())                        # [B, C, S]
    if has_init is not None:
        prev = prev * has_init.to(prev.dtype).view(b, 1, 1)
    xf = x.float()
    acc = torch.zeros(t, c, dtype=torch.float32, device=dev)
    for j in range(k):
        back = (k - 1 - j) * dilation                                    # rows between this tap and the current row
        src = local - back
        inside = src >= 0
        from_x = xf[(start + src).clamp_(min=0)]
        from_w = prev[seq, :, (s + src).clamp_(min=0, max=max(s - 1, 0))].float() if s else torch.zeros_like(from_x)
        acc += weight[:, j].float() * torch.where(inside[:, None], from_x, from_w)
    # windows after the rows: the last S rows of [previous window | the sequence's rows]
    if s == 0:
        return acc.to(x.dtype)
    first = rows if q_indptr is None else q_indptr.long()[:-1]           # first row of every sequence, [B]
    pos = length[:, None] + torch.arange(s, device=dev)[None, :]         # index into the concatenation, [B, S]
    old = prev.gather(2, pos.clamp(max=s - 1)[:, None, :].expand(b, c, s))
    new_rows = x[(first[:, None] + (pos - s)).clamp_(min=0, max=t - 1)]  # [B, S, C]
    new = torch.where((pos < s)[:, None, :], old, new_rows.transpose(1, 2).to(window.dtype))
    window.index_copy_(0, slot_out.long(), new)
    return acc.to(x.dtype)


class PleLayer:
    """Per-layer n-gram embedding added to the hyper-connection streams before a block (Flash-Next: block 1).

    Every token reads `heads` rows of an fp8 table, picked by hashes of its trailing 2- and 3-grams; the rows are
    projected to a key per stream and one value, the key scores the stream's current content, the gated value goes
    through a dilated depth-wise convolution over time and is added to the streams. The layer's state per sequence
    is the convolution window and the two last tokens (the n-gram context of the next token); both live in the
    recurrent-state pool as auxiliary tensors, so prefix snapshots, scratch slots of speculative verification and
    replay of the accepted rows treat them like any other recurrent state, and the token history never needs the
    host. Reference: hibana/model/flashnext/ple.py:205-399 (PleLayer), :250-277 (the hash).
    """

    STATE_WINDOW, STATE_HISTORY = "ple_window", "ple_history"

    def __init__(self, t, init, name: str, table: Optional[PleTable] = None):
        self.t, self.name = t, name
        self.hc, self.hidden, self.eps = max(t.hyper_streams, 1), t.hidden, t.norm_eps
        self.ngram, self.per, self.kernel = 3, t.ple_heads, t.ple_kernel
        self.heads = (self.ngram - 1) * self.per
        self.dim = self.heads * ROW_DIM
        self.eos = t.ple_eos
        dev = init.device
        self.key_proj = init.linear(self.hc * self.hidden, self.dim, "bf16", name + ".key_proj")
        self.value_proj = init.linear(self.hidden, self.dim, "bf16", name + ".value_proj")
        width = self.hc * self.hidden
        self.norm_key = torch.zeros(width, dtype=torch.bfloat16, device=dev)
        self.norm_query = torch.zeros(width, dtype=torch.bfloat16, device=dev)
        self.norm_conv = torch.zeros(width, dtype=torch.bfloat16, device=dev)
        self.conv_weight = init.normal(width, self.kernel, std=0.3).to(torch.bfloat16).to(dev)
        # hash parameters (part of the checkpoint): one odd multiplier per n-gram position, a vocabulary per head,
        # the heads' row ranges back to back in the table
        self.multipliers = (init.uniform(self.ngram, lo=float(1 << 20), hi=float(1 << 40)).long() | 1).to(dev)
        sizes = [t.ple_rows - 2 * i - 1 for i in range(self.heads)]
        self.vocab_sizes = torch.tensor(sizes, dtype=torch.int64, device=dev)
        self.offsets = torch.tensor([sum(sizes[:i]) for i in range(self.heads)], dtype=torch.int64, device=dev)
        self.scale = 0.05
        if table is None:       # synthetic table, resident on the device
            rows = sum(sizes)
            self.rows = torch.cat([(init.normal(min(1 << 16, rows - r0), ROW_DIM, std=2.0)).to(torch.float8_e4m3fn)
                                   .view(torch.uint8).to(dev) for r0 in range(0, rows, 1 << 16)])
            self.table = None
        else:
            self.rows, self.table = None, table
        self._scratch = None

    # ---- state
    def register(self, pool) -> None:
        s = (self.kernel - 1) * self.ngram
        pool.register_aux(self.STATE_WINDOW, (self.hc * self.hidden, s), torch.bfloat16)
        pool.register_aux(self.STATE_HISTORY, (2,), torch.int64, fill=self.eos)

    def _state(self, states, dev):
        if states is not None:
            self.register(states)
            return states.aux[self.STATE_WINDOW], states.aux[self.STATE_HISTORY]
        if self._scratch is None:       # stand-alone use (no pool): slot 0 only
            s = (self.kernel - 1) * self.ngram
            self._scratch = (torch.zeros(1, self.hc * self.hidden, s, dtype=torch.bfloat16, device=dev),
                             torch.full((1, 2), self.eos, dtype=torch.int64, device=dev))
        return self._scratch

    # ---- table rows
    def row_ids(self, cur: torch.Tensor, back1: torch.Tensor, back2: torch.Tensor) -> torch.Tensor:
        """int64 [N] each -> table rows int64 [N, heads]. An end-of-sequence token cuts the context: what lies
        behind it counts as end-of-sequence too."""
        eos = self.eos
        back2 = torch.where((back1 == eos) | (back2 == eos), torch.full_like(back2, eos), back2)
        m = self.multipliers
        mix2 = (cur * m[0]) ^ (back1 * m[1])
        mix3 = mix2 ^ (back2 * m[2])
        p = self.per
        two = torch.remainder(mix2[:, None], self.vocab_sizes[None, :p]) + self.offsets[None, :p]
        three = torch.remainder(mix3[:, None], self.vocab_sizes[None, p:]) + self.offsets[None, p:]
        return torch.cat((two, three), dim=1)

    def _contexts(self, ids: torch.Tensor, hist: torch.Tensor, q_indptr, has_init, seq, local, start):
        """The two tokens before every row: earlier rows of the same sequence, else the slot's stored history."""
        t = ids.shape[0]
        prev = hist if has_init is None else torch.where(has_init.bool()[:, None], hist, torch.full_like(hist, self.eos))
        idx = torch.arange(t, device=ids.device)
        b1 = torch.where(local >= 1, ids[(idx - 1).clamp_(min=0)], prev[seq, 1])
        b2 = torch.where(local >= 2, ids[(idx - 2).clamp_(min=0)], torch.where(local == 1, prev[seq, 1], prev[seq, 0]))
        return b1, b2

    def forward(self, hyper: torch.Tensor, ids: torch.Tensor, ctx, states=None) -> torch.Tensor:
        """hyper [T, hc * H] bf16, ids int64 [T] -> the addend for `hyper` (same shape, bf16)."""
        t, dev = hyper.shape[0], hyper.device
        window, history = self._state(states, dev)
        b = ctx.state_slots.shape[0] if ctx is not None and ctx.state_slots is not None else 1
        slot_in = ctx.state_slots.long() if ctx is not None and ctx.state_slots is not None else torch.zeros(1, dtype=torch.int64, device=dev)
        slot_out = slot_in
        q_indptr = has_init = None
        if ctx is not None:
            so = ctx.extras.get("state_out")
            slot_out = so.long() if so is not None else slot_in
            q_indptr, has_init = ctx.q_indptr, ctx.has_initial_state
        rows = torch.arange(t, device=dev)
        if q_indptr is None and b == t:
            seq, local, start = rows, torch.zeros_like(rows), rows
            last = rows
        else:
            ip = q_indptr.long() if q_indptr is not None else torch.tensor([0, t], device=dev)
            seq = torch.bucketize(rows, ip[1:], right=True).clamp_(max=b - 1)
            start = ip[:-1][seq]
            local = rows - start
            last = ip[1:] - 1
            if q_indptr is None:
                q_indptr = ip.to(torch.int32)
        hist_in = history.index_select(0, slot_in)
        b1, b2 = self._contexts(ids, hist_in, q_indptr, has_init, seq, local, start)
        table_rows = self.row_ids(ids, b1, b2)
        raw = (self.rows.index_select(0, table_rows.reshape(-1)) if self.rows is not None
               else self.table.gather(table_rows.cpu().numpy()).to(dev).view(-1, ROW_DIM))
        emb = (raw.view(torch.float8_e4m3fn).to(torch.bfloat16) * self.scale).view(t, self.dim)
        key = self.key_proj(emb)
        value = self.value_proj(emb)
        key_n = gemma_group_norm(key, self.norm_key, self.hc, self.eps).view(t, self.hc, self.hidden)
        query_n = gemma_group_norm(hyper, self.norm_query, self.hc, self.eps).view(t, self.hc, self.hidden)
        gate = (key_n.float() * query_n.float()).sum(-1, keepdim=True) / (self.hidden ** 0.5)
        gate = torch.sigmoid(gate.abs().clamp_min(1e-6).sqrt() * gate.sign())
        gated = (gate * value.float().unsqueeze(1)).flatten(1)                     # [T, hc * H] fp32
        gated_n = gemma_group_norm(gated.to(torch.bfloat16), self.norm_conv, self.hc, self.eps)
        if ctx is not None and "ring" in ctx.extras:       # verify: log what the accepted rows have to replay
            ctx.extras["ring"].append((self, (gated_n, ids)))
        conv = dilated_conv_ragged(gated_n, self.conv_weight, self.ngram, window, slot_in, slot_out, q_indptr, has_init)
        self._advance_history(history, ids, hist_in, slot_out, last, has_init, q_indptr)
        return (gated + torch.nn.functional.silu(conv.float())).to(hyper.dtype)

    def _advance_history(self, history, ids, hist_in, slot_out, last, has_init, q_indptr) -> None:
        """The two last tokens of every sequence after its rows."""
        prev = hist_in if has_init is None else torch.where(has_init.bool()[:, None], hist_in,
                                                            torch.full_like(hist_in, self.eos))
        if q_indptr is None:
            length = torch.ones_like(last)
        else:
            ip = q_indptr.long()
            length = ip[1:] - ip[:-1]
        newest = ids[last.clamp(min=0)]
        before = torch.where(length >= 2, ids[(last - 1).clamp(min=0)], prev[:, 1])
        new = torch.stack((torch.where(length >= 1, before, prev[:, 0]), torch.where(length >= 1, newest, prev[:, 1])), 1)
        history.index_copy_(0, slot_out, new)

    def replay(self, saved, sel, q_indptr, slots, states) -> None:
        """Advances the committed window and history over the accepted rows of a verify block."""
        window, history = self._state(states, saved[0].device)
        x, ids = saved[0].index_select(0, sel), saved[1].index_select(0, sel)
        sl = slots.long()
        dilated_conv_ragged(x, self.conv_weight, self.ngram, window, sl, sl, q_indptr, None)
        ip = q_indptr.long()
        self._advance_history(history, ids, history.index_select(0, sl), sl, ip[1:] - 1, None, q_indptr)

    def weight_bytes(self) -> int:
        table = self.rows.numel() if self.rows is not None else 0
        return self.key_proj.nbytes() + self.value_proj.nbytes() + table + self.conv_weight.numel() * 2
