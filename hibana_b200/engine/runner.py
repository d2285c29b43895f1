"""Device-side step mechanics: block table, one packed upload per step, CUDA-graph decode buckets.

The runner knows nothing about requests. The executor hands it rows of the device block table, token ids,
positions and KV slots; it uploads them in one pinned copy, runs the model (a captured graph for decode
buckets, eager for prefill chunks), samples on the device and reads back one small tensor.
Reference counterparts: hibana/engine/graphs.py:45-159 (one graph per batch bucket, static buffers, padded
rows to slot 0) and hibana/engine/upload.py (pinned non-blocking upload).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import _native as nv
from .. import config as cfgmod
from ..ops import attention, sampling
from .context import DECODE, PREFILL, VERIFY, ForwardContext

# Rows of the packed int32 step buffer.
R_IDS, R_POS, R_SLOT, R_ROW, R_CTX, R_TOPK, R_TEMP, R_TOPP, R_SEED, R_OFFS, R_STATE, N_ROWS = \
    0, 1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 13


class StepBuffers:
    """Static device buffers + pinned staging of one decode bucket."""

    def __init__(self, bucket: int, device: torch.device):
        self.bucket = bucket
        self.dev = torch.zeros(N_ROWS, bucket, dtype=torch.int32, device=device)
        pin = device.type == "cuda"
        self.host = torch.zeros(N_ROWS, bucket, dtype=torch.int32, pin_memory=pin)
        self.np = self.host.numpy()
        self.out = torch.zeros(bucket, dtype=torch.int64, device=device)
        self.out_host = torch.zeros(bucket, dtype=torch.int64, pin_memory=pin)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_greedy: Optional[torch.cuda.CUDAGraph] = None   # tensor parallel: greedy-only step (no logits gather)
        self.workspace = None
        self.splits = 1
        self.mask: Optional[torch.Tensor] = None      # grammar bitmask [bucket, ceil(vocab / 32)], all ones = free
        self.mask_dirty: list = []

    def views(self):
        d = self.dev
        flat = d.view(-1)
        b = self.bucket
        return dict(ids=d[R_IDS], pos=d[R_POS], slot=d[R_SLOT], row=d[R_ROW], ctx=d[R_CTX], top_k=d[R_TOPK],
                    state=d[R_STATE],
                    temp=d[R_TEMP].view(torch.float32), top_p=d[R_TOPP].view(torch.float32),
                    seed=flat[R_SEED * b:(R_SEED + 2) * b].view(torch.int64),
                    offs=flat[R_OFFS * b:(R_OFFS + 2) * b].view(torch.int64))


class ModelRunner:
    def __init__(self, model, kv_pool, *, max_batch: int, max_ctx: int, buckets: Sequence[int] = (1, 2, 4, 8, 16, 32, 64),
                 use_graphs: bool = True, state_pool=None, comm=None, attn_splits: int = 0):
        self.model, self.kv, self.state_pool, self.comm = model, kv_pool, state_pool, comm
        self.device = model.device
        self.max_batch, self.max_ctx = max_batch, max_ctx
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self.attn_splits = attn_splits
        # Row 0 is the dummy sequence padded graph rows point at.
        self.block_table = torch.zeros(max_batch + 1, max_ctx, dtype=torch.int32, device=self.device)
        self._free_rows = list(range(max_batch, 0, -1))
        self.buckets = tuple(sorted(b for b in buckets if b <= max_batch)) or (max_batch,)
        if self.buckets[-1] < max_batch:
            self.buckets = self.buckets + (max_batch,)
        self.bufs = {b: StepBuffers(b, self.device) for b in self.buckets}
        self.graph_launches: dict[int, int] = {}   # kernels of this library inside each bucket's graph
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # The device status word travels to the host with every step's sampled tokens (same stream, same
        # synchronize): a bounded wait that gave up anywhere in the step voids it, and every later collective
        # would give up at once, so the step raises instead of streaming garbage.
        self._status_dev = nv.device_state(self.device).status if self.device.type == "cuda" else None
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=self.device.type == "cuda")

    def _queue_status_read(self) -> None:
        if self._status_dev is not None:
            self._status_host.copy_(self._status_dev[:1], non_blocking=True)

    def _raise_on_status(self) -> None:
        """Call after the synchronize that follows `_queue_status_read`."""
        code = int(self._status_host[0]) if self._status_dev is not None else 0
        if code:
            self._status_dev.zero_()
            self._status_host.zero_()
            raise nv.DeviceWaitTimeout(code)

    # ---- block table rows
    def alloc_row(self) -> int:
        if not self._free_rows:
            raise MemoryError("no free block-table row")
        return self._free_rows.pop()

    def free_row(self, row: int) -> None:
        if row > 0:
            self._free_rows.append(row)

    def set_table(self, row: int, start: int, slots: Sequence[int]) -> None:
        """Writes slots of positions [start, start + len) of a sequence (cache hits, restores)."""
        if not len(slots):
            return
        t = torch.tensor(list(slots), dtype=torch.int32)
        if self.device.type == "cuda":
            t = t.pin_memory()
        self.block_table[row, start:start + len(slots)].copy_(t, non_blocking=True)
        self.h2d_bytes += t.numel() * 4

    # ---- decode
    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        raise ValueError(f"batch {n} exceeds the largest bucket {self.buckets[-1]}")

    def _decode_body(self, buf: StepBuffers, greedy: bool = False) -> None:
        """`greedy`: every row is greedy and unconstrained; with a vocab-parallel head the ranks then exchange one
        (value, id) pair per row instead of gathering the logits."""
        v = buf.views()
        self.block_table.index_put_((v["row"].long(), v["pos"].long()), v["slot"])
        ctx = ForwardContext(DECODE, positions=v["pos"], slots=v["slot"], kv_indices=self.block_table,
                             ctx_len=v["ctx"], seq_rows=v["row"], batch=buf.bucket, attn_splits=buf.splits,
                             attn_workspace=buf.workspace, comm=self.comm,
                             state_slots=v["state"])
        h = self._forward(v["ids"].long(), ctx)
        if greedy:
            buf.out.copy_(self.model.greedy_tokens(h, self.comm))
            return
        logits = self.model.logits(h, self.comm) if self.comm is not None else self.model.logits(h)
        buf.logits = logits          # stable inside a captured graph: read back only for requests that want logprobs
        tok = sampling.sample(logits, v["temp"], v["top_k"], v["top_p"], v["seed"], v["offs"], bitmask=buf.mask)
        buf.out.copy_(tok)

    def _prepare_bucket(self, buf: StepBuffers) -> None:
        t = self.model.target
        if buf.workspace is None and t.attn_layers:
            buf.splits = self.attn_splits or attention.choose_splits(buf.bucket, t.kv_heads, self.max_ctx)
            if buf.splits > 1 and self.device.type == "cuda":
                buf.workspace = attention.AttnWorkspace(buf.bucket, t.q_heads, t.head_dim, buf.splits, self.device)
        if buf.mask is None:      # read by the sampling kernels next to the logits; rows of constrained requests
            buf.mask = torch.full((buf.bucket, (t.vocab + 31) // 32), -1, dtype=torch.int32, device=self.device)

    def capture(self, buckets: Optional[Sequence[int]] = None) -> None:
        """Captures one decode graph per bucket (after a warm-up run of the same body)."""
        if not self.use_graphs:
            return
        for b in (buckets or self.buckets):
            buf = self.bufs[b]
            self._prepare_bucket(buf)
            buf.dev.zero_()
            buf.dev[R_CTX].fill_(1)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_body(buf)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = nv.LAUNCHES
            with torch.cuda.graph(g):
                self._decode_body(buf)
            self.graph_launches[b] = nv.LAUNCHES - before
            buf.graph = g
            if self._split_head():
                with torch.cuda.stream(s):
                    self._decode_body(buf, greedy=True)
                torch.cuda.current_stream().wait_stream(s)
                torch.cuda.synchronize()
                g2 = torch.cuda.CUDAGraph()
                before = nv.LAUNCHES
                with torch.cuda.graph(g2):
                    self._decode_body(buf, greedy=True)
                self.graph_launches[b] = nv.LAUNCHES - before     # the common step: report this one
                buf.graph_greedy = g2

    def _split_head(self) -> bool:
        return (self.comm is not None and getattr(self.model, "vocab_shard", 0) > 0
                and hasattr(self.model, "greedy_tokens") and hasattr(self.comm, "pick_exchange"))

    debug_sync = False      # synchronise and read the status word after every forward (slow; pins a fault to it)
    qsa = False             # sparse-attention indexer in use (the target has one and contexts can exceed its budget)
    ep = None               # expert-parallel all-to-all handle (parallel/ep.py): MoE layers exchange rows through it
    lockstep = None         # engine/dp.py Lockstep: data-parallel ranks align their forwards through it
    _in_round = False

    def _enter_forward(self) -> None:
        """Data-parallel ranks with expert-parallel layers run every forward together: announce this one."""
        if self.lockstep is not None and not self._in_round:
            from .dp import FORWARD
            self.lockstep.round(FORWARD)

    def idle_round(self, state: int = 0) -> list:
        """A round for a rank with nothing to run: joins the others' forward with an empty batch when there is
        one. Returns what every rank posted."""
        from .dp import FORWARD
        states = self.lockstep.round(state)
        if FORWARD in states and self.ep is not None:
            self._in_round = True
            try:
                self.decode([], [], [], [])
            finally:
                self._in_round = False
            self.lockstep.empty_forwards += 1
        return states

    def _forward(self, ids, ctx):
        if self.ep is not None:
            ctx.extras["ep"] = self.ep
        if self.qsa:
            ctx.extras["qsa"], ctx.extras["qsa_max_pos"] = True, self.max_ctx
        if self.state_pool is not None:
            h = self.model.forward(ids, ctx, self.kv, self.state_pool)
        else:
            h = self.model.forward(ids, ctx, self.kv)
        if self.debug_sync and self.device.type == "cuda" and not torch.cuda.is_current_stream_capturing():
            torch.cuda.synchronize(self.device)
            code = nv.read_status(self.device)
            if code:
                raise nv.DeviceWaitTimeout(code)
        return h

    def decode(self, rows: Sequence[int], tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int],
               sampling_rows: Optional[dict] = None, state_slots: Optional[Sequence[int]] = None,
               masks: Optional[Sequence] = None, logprobs: Optional[Sequence[int]] = None) -> list[int]:
        """One decode step for len(rows) sequences; returns the sampled token of each (host ints).
        `masks[i]` (host int32 [ceil(vocab / 32)] or None) restricts sequence i's token to a grammar.
        `logprobs[i]` > 0 asks for the log-probability of sequence i's token and its top-k alternatives; they are
        left in `self.last_logprobs[i]` = (logprob, [(token, logprob), ...]).

        sampling_rows: optional dict of per-sequence lists temp / top_k / top_p / seed / offs (greedy when None).
        """
        n = len(rows)
        self._enter_forward()
        buf = self.bufs[self._bucket(n)]
        self._prepare_bucket(buf)
        a = buf.np
        a[:, n:] = 0
        a[R_CTX, n:] = 1
        a[R_IDS, :n] = tokens
        a[R_POS, :n] = positions
        a[R_SLOT, :n] = slots
        a[R_ROW, :n] = rows
        a[R_CTX, :n] = np.asarray(positions, dtype=np.int32) + 1
        if state_slots is not None:
            a[R_STATE, :n] = state_slots
        if sampling_rows is None:
            a[R_TOPK:R_OFFS + 2, :n] = 0
        else:
            a[R_TOPK, :n] = sampling_rows["top_k"]
            a[R_TEMP].view(np.float32)[:n] = sampling_rows["temp"]
            a[R_TOPP].view(np.float32)[:n] = sampling_rows["top_p"]
            a[R_SEED:R_SEED + 2].reshape(-1).view(np.int64)[:n] = sampling_rows["seed"]
            a[R_OFFS:R_OFFS + 2].reshape(-1).view(np.int64)[:n] = sampling_rows["offs"]
        buf.dev.copy_(buf.host, non_blocking=True)
        self.h2d_bytes += buf.host.numel() * 4
        for i in buf.mask_dirty:           # rows a previous step constrained are free again
            buf.mask[i].fill_(-1)
        buf.mask_dirty = []
        if masks is not None:
            for i, m in enumerate(masks):
                if m is not None:
                    buf.mask[i].copy_(m, non_blocking=True)
                    buf.mask_dirty.append(i)
                    self.h2d_bytes += m.numel() * 4
        want_lp = logprobs is not None and any(logprobs)
        greedy = sampling_rows is None and masks is None and self._split_head() and not want_lp
        if greedy and buf.graph_greedy is not None:
            buf.graph_greedy.replay()
        elif buf.graph is not None:
            buf.graph.replay()
        else:
            self._decode_body(buf, greedy=greedy)
        buf.out_host.copy_(buf.out, non_blocking=True)
        self._queue_status_read()
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.d2h_bytes += buf.bucket * 8 + (4 if self._status_dev is not None else 0)
        self._raise_on_status()
        self.last_logprobs = self._logprobs(buf.logits, buf.out, logprobs, n) if want_lp else None
        return buf.out_host[:n].tolist()

    last_logprobs = None

    def _logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, ks: Sequence[int], n: int) -> dict:
        """{row: (logprob of its token, [(token, logprob)] of its ks[row] most likely tokens)} for rows with k > 0."""
        idx = [i for i in range(n) if ks[i]]
        sel = torch.tensor(idx, dtype=torch.long, device=logits.device)
        lp = torch.log_softmax(logits.index_select(0, sel).float(), dim=-1)
        chosen = lp.gather(1, tokens.index_select(0, sel).view(-1, 1)).squeeze(1).tolist()
        kmax = min(max(ks[i] for i in idx), lp.shape[1])
        topv, topi = lp.topk(kmax, dim=-1)
        topv, topi = topv.tolist(), topi.tolist()
        return {i: (chosen[j], list(zip(topi[j][:ks[i]], topv[j][:ks[i]]))) for j, i in enumerate(idx)}

    # ---- prefill / verify (eager, ragged)
    def forward_rows(self, rows: Sequence[int], token_lists: Sequence[Sequence[int]], starts: Sequence[int],
                     slot_lists: Sequence[Sequence[int]], *, mode: str = PREFILL, want: str = "last",
                     sampling_rows: Optional[dict] = None, state_slots: Optional[Sequence[int]] = None,
                     has_initial_state: Optional[Sequence[int]] = None, checkpoints=None,
                     extras: Optional[dict] = None, masks: Optional[torch.Tensor] = None,
                     logprobs: Optional[Sequence[int]] = None):
        """Runs new tokens of several sequences in one ragged forward.

        rows[i] is the block-table row, token_lists[i] the new tokens starting at position starts[i] with KV slots
        slot_lists[i]. want='last' samples one token per sequence from its last row, 'all' returns the argmax of
        every row (verify), 'none' skips the head. Returns a host list (or None).
        """
        dev = self.device
        self._enter_forward()
        counts = [len(t) for t in token_lists]
        total = sum(counts)
        b = len(rows)
        ids = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists])
        pos = np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(starts, counts)])
        slots = np.concatenate([np.asarray(s, dtype=np.int32) for s in slot_lists])
        tok_rows = np.repeat(np.asarray(rows, dtype=np.int64), counts)
        indptr = np.zeros(b + 1, dtype=np.int32)
        indptr[1:] = np.cumsum(counts)
        ctx_len = np.asarray([s + c for s, c in zip(starts, counts)], dtype=np.int32)
        pin = dev.type == "cuda"

        def up(arr, dtype):
            t = torch.from_numpy(np.ascontiguousarray(arr)).to(dtype)
            if pin:
                t = t.pin_memory()
            self.h2d_bytes += t.numel() * t.element_size()
            return t.to(dev, non_blocking=True)

        ids_d, pos_d, slots_d = up(ids, torch.int64), up(pos, torch.int32), up(slots, torch.int32)
        rows_d, indptr_d, ctx_d = up(tok_rows, torch.int64), up(indptr, torch.int32), up(ctx_len, torch.int32)
        seq_rows_d = up(np.asarray(rows, dtype=np.int32), torch.int32)
        self.block_table.index_put_((rows_d, pos_d.long()), slots_d)
        last = torch.from_numpy(indptr[1:].astype(np.int64) - 1).to(dev) if want == "last" else None
        t = self.model.target
        max_rows = max(counts)
        splits = 1
        if cfgmod.current().stable_numerics:
            pass
        elif t.attn_layers and b * t.kv_heads * max(1, max_rows // max(1, 32 // max(1, t.q_heads // max(t.kv_heads, 1)))) < 148:
            splits = attention.choose_splits(b, t.kv_heads, int(ctx_len.max()))
        ctx = ForwardContext(mode, positions=pos_d, slots=slots_d, kv_indices=self.block_table, ctx_len=ctx_d,
                             q_indptr=indptr_d, seq_rows=seq_rows_d, max_rows=max_rows, batch=b, sample_rows=last,
                             attn_splits=splits, comm=self.comm, seq_starts_host=list(counts),
                             state_slots=up(np.asarray(state_slots, dtype=np.int32), torch.int32)
                             if state_slots is not None else seq_rows_d,
                             has_initial_state=up(np.asarray(has_initial_state, dtype=np.int32), torch.int32)
                             if has_initial_state is not None else None,
                             checkpoints=checkpoints, max_ctx_host=int(ctx_len.max()),
                             extras=extras if extras is not None else {})
        h = self._forward(ids_d, ctx)
        if want == "none":
            return None
        if want in ("all_device", "logits_device"):
            # verify: argmax (or the logits themselves, for relaxed / sampled acceptance) of every row and the
            # pre-norm hidden states, left on the device
            logits = self.model.logits(h, self.comm) if self.comm is not None else self.model.logits(h)
            return (logits if want == "logits_device" else sampling.argmax(logits)), ctx.extras.get("hidden")
        logits = self.model.logits(h, self.comm) if self.comm is not None else self.model.logits(h)
        if masks is not None:      # grammar bitmask per sampled row (host int32 [rows, ceil(vocab / 32)])
            masks = masks.to(dev, non_blocking=True)
        if sampling_rows is None or want == "all":
            tok = sampling.argmax(logits, masks if want == "last" else None)
        else:
            sr = {k: up(np.asarray(v), dt) for (k, v), dt in zip(
                ((k, sampling_rows[k]) for k in ("temp", "top_k", "top_p", "seed", "offs")),
                (torch.float32, torch.int32, torch.float32, torch.int64, torch.int64))}
            tok = sampling.sample(logits, sr["temp"], sr["top_k"], sr["top_p"], sr["seed"], sr["offs"], bitmask=masks)
        self.last_logprobs = (self._logprobs(logits, tok, logprobs, b)
                              if want == "last" and logprobs is not None and any(logprobs) else None)
        self._queue_status_read()
        out = tok.cpu()         # synchronises the stream: the status word queued before it has landed too
        self.d2h_bytes += out.numel() * 8 + (4 if self._status_dev is not None else 0)
        self._raise_on_status()
        return out.tolist()
