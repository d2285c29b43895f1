"""CUDA-graph verify + device-resident accept for speculative rounds.

A speculative round's verify forward runs k + 1 rows per request (the pending token and k drafted tokens). Run
eagerly it costs hundreds of host-launched kernels plus numpy packing and several small uploads; here it is one
captured graph per (batch bucket, depth):

    one pinned upload (token-level rows: ids / positions / KV slots / block-table rows; request-level rows: table
    row, context length, token budget, stop ids)
      -> graph: block-table update, ragged verify forward (uniform k + 1 rows per request, static q_indptr),
         lm_head, argmax of every row, the accept kernel (longest exact prefix + the target's own token, cut at
         stop ids and the budget)
      -> one readback of META = [emitted tokens | count | accepted] per request.

The verified hidden states stay on the device for the drafter (MTP feature of the last accepted row). Padded
requests of a bucket point at block-table row 0 / KV slot 0, as in the decode graphs. On a CPU device the same
body runs eagerly over the same static buffers, which is what the CPU tests compare with the host round.
Covers greedy and sampled requests (the rejection-sampling rule against the deterministic drafts is one kernel
after the head, ops/sampling.py `spec_targets`; greedy requests keep their argmax) of unconstrained requests, on
models with recurrent layers too: the verify forward writes its end state to a scratch slot per request row and
logs every recurrent layer's inputs, and after the accept kernel the same graph replays the accepted rows into the
requests' own state slots, the row selection and row pointers derived from the device-side counts. Relaxed-greedy
acceptance and grammar masks take the eager round. Reference: hibana/engine/spec_graphs.py:43-164
(VerifyGraphs), hibana/engine/accept_graphs.py:50-310 (AcceptGraphs), hibana/proposers/mtp_graphs.py:15 (DraftGraphs).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import _native as nv
from ..ops import attention, sampling
from .context import VERIFY, ForwardContext
from .request import MAX_STOPS

T_IDS, T_POS, T_SLOT, T_ROW, T_FIELDS = 0, 1, 2, 3, 4          # token-level rows
# request-level rows: table row, context length, token budget, sampling parameters (seed and draw counter are
# 64-bit: two rows each, on an even row so that the pair is 8-byte aligned for every bucket), the request's
# recurrent-state slot, then the stop ids
S_ROW, S_CTX, S_BUDGET, S_TOPK, S_SEED, S_DRAWS, S_TEMP, S_TOPP, S_SOFT, S_STATE, S_STOP0 = 0, 1, 2, 3, 4, 6, 8, 9, 10, 11, 12


class VerifyBuffers:
    def __init__(self, bucket: int, k1: int, device: torch.device):
        self.bucket, self.k1 = bucket, k1
        rows = bucket * k1
        self.n_tok, self.n_seq = T_FIELDS * rows, (S_STOP0 + MAX_STOPS) * bucket
        pin = device.type == "cuda"
        self.host = torch.zeros(self.n_tok + self.n_seq, dtype=torch.int32, pin_memory=pin)
        self.np = self.host.numpy()
        self.dev = torch.zeros(self.n_tok + self.n_seq, dtype=torch.int32, device=device)
        self.tok = self.dev[:self.n_tok].view(T_FIELDS, rows)
        self.seq = self.dev[self.n_tok:].view(S_STOP0 + MAX_STOPS, bucket)
        self.tok_np = self.np[:self.n_tok].reshape(T_FIELDS, rows)
        self.seq_np = self.np[self.n_tok:].reshape(S_STOP0 + MAX_STOPS, bucket)
        self.indptr = (torch.arange(bucket + 1, dtype=torch.int32) * k1).to(device)
        self.meta = torch.zeros(bucket, k1 + 2, dtype=torch.int64, device=device)
        self.meta_host = torch.zeros(bucket, k1 + 2, dtype=torch.int64, pin_memory=pin)
        self.hidden: Optional[torch.Tensor] = None      # [bucket * k1, H] pre-norm hidden of every verified row
        self.graph = None
        self.workspace = None
        self.splits = 1
        self.scratch: Optional[torch.Tensor] = None     # recurrent models: one scratch state slot per request row


class VerifyGraphs:
    def __init__(self, runner, depth: int, buckets: Optional[Sequence[int]] = None):
        self.runner, self.model = runner, runner.model
        self.k1 = depth + 1
        self.device = runner.device
        self.buckets = tuple(buckets or runner.buckets)
        self.bufs = {b: VerifyBuffers(b, self.k1, self.device) for b in self.buckets}
        self.launches: dict = {}
        self.rounds = 0
        self._scratch: Optional[torch.Tensor] = None

    def supported(self) -> bool:
        """Attention-only models always; recurrent models when the state pool can spare one scratch slot per row
        of the largest bucket (the verify forward writes the state after its k + 1 rows there, the accepted prefix
        is then replayed into the request's own slot inside the same graph)."""
        pool = self.runner.state_pool
        return pool is None or pool.free_count > 2 * max(self.buckets)

    # ---- the captured body
    def _body(self, buf: VerifyBuffers) -> None:
        r = self.runner
        b, k1 = buf.bucket, buf.k1
        tok, seq = buf.tok, buf.seq
        r.block_table.index_put_((tok[T_ROW].long(), tok[T_POS].long()), tok[T_SLOT])
        extras = {"want_hidden": True}
        if buf.scratch is not None:
            extras["state_out"], extras["ring"] = buf.scratch, []
        ctx = ForwardContext(VERIFY, positions=tok[T_POS], slots=tok[T_SLOT], kv_indices=r.block_table,
                             ctx_len=seq[S_CTX], q_indptr=buf.indptr, seq_rows=seq[S_ROW], max_rows=k1, batch=b,
                             attn_splits=buf.splits, attn_workspace=buf.workspace, comm=r.comm,
                             seq_starts_host=[k1] * b, state_slots=seq[S_STATE], extras=extras)
        h = r._forward(tok[T_IDS].long(), ctx)
        buf.hidden = ctx.extras.get("hidden")
        logits = self.model.logits(h, r.comm) if r.comm is not None else self.model.logits(h)
        drafts = tok[T_IDS].view(b, k1)[:, 1:].long().contiguous()
        pick = sampling.argmax(logits)
        target, _ = sampling.spec_targets(
            logits, drafts, seq[S_TEMP].view(torch.float32), seq[S_TOPK], seq[S_TOPP].view(torch.float32),
            seq[S_SEED:S_SEED + 2].reshape(-1).view(torch.int64)[:b],
            seq[S_DRAWS:S_DRAWS + 2].reshape(-1).view(torch.int64)[:b], seq[S_SOFT].view(torch.float32),
            greedy_pick=pick)
        stops = seq[S_STOP0:S_STOP0 + MAX_STOPS].t().long().contiguous()
        emitted, count, accepted = sampling.accept_greedy(target, drafts, stops, seq[S_BUDGET].contiguous())
        buf.meta[:, :k1].copy_(emitted)
        buf.meta[:, k1].copy_(count)
        buf.meta[:, k1 + 1].copy_(accepted)
        if buf.scratch is not None:
            # commit the recurrent state of the accepted prefix without asking the host how long it is: the rows a
            # request keeps are its first count[i]; a scatter packs them to the front in request order, the row
            # pointers are the running sum of the counts, and every recurrent layer replays its logged inputs over
            # exactly those rows into the request's own state slot
            cnt = count.to(torch.int32)
            ip = torch.zeros(b + 1, dtype=torch.int32, device=cnt.device)
            ip[1:] = torch.cumsum(cnt, 0)
            j = torch.arange(k1, device=cnt.device)[None, :]
            dest = torch.where(j < cnt[:, None], ip[:-1, None] + j, b * k1).reshape(-1).long()
            sel = torch.zeros(b * k1 + 1, dtype=torch.int64, device=cnt.device)
            sel.scatter_(0, dest, torch.arange(b * k1, device=cnt.device))      # dropped rows land in the spare cell
            sel = sel[:b * k1]
            for layer, saved in extras["ring"]:
                layer.replay(saved, sel, ip, seq[S_STATE], r.state_pool)

    def _prepare(self, buf: VerifyBuffers) -> None:
        t = self.model.target
        pool = self.runner.state_pool
        if pool is not None and buf.scratch is None:
            if self._scratch is None:                       # one set of scratch slots, shared by every bucket
                self._scratch = torch.tensor(pool.reserve(max(self.buckets)), dtype=torch.int32,
                                             device=self.device)
            buf.scratch = self._scratch[:buf.bucket]
        if buf.workspace is None and t.attn_layers and self.device.type == "cuda":
            buf.splits = self.runner.attn_splits or attention.choose_splits(buf.bucket, t.kv_heads, self.runner.max_ctx,
                                                                            row_chunks=1)
            if buf.splits > 1:
                buf.workspace = attention.AttnWorkspace(buf.bucket * buf.k1, t.q_heads, t.head_dim, buf.splits,
                                                        self.device)

    def capture(self) -> None:
        if self.device.type != "cuda" or not self.runner.use_graphs:
            return
        for b, buf in self.bufs.items():
            self._prepare(buf)
            buf.dev.zero_()
            buf.seq[S_CTX].fill_(buf.k1)
            buf.seq[S_BUDGET].fill_(1)
            buf.tok[T_POS].copy_(torch.arange(buf.k1, dtype=torch.int32, device=self.device).repeat(b))
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._body(buf)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = nv.LAUNCHES
            with torch.cuda.graph(g):
                self._body(buf)
            self.launches[b] = nv.LAUNCHES - before
            buf.graph = g

    # ---- one round
    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        raise ValueError(f"batch {n} exceeds the largest verify bucket {self.buckets[-1]}")

    def run(self, rows: Sequence[int], tokens: Sequence[Sequence[int]], starts: Sequence[int],
            slot_lists: Sequence[Sequence[int]], stop_lists: Sequence[Sequence[int]], budgets: Sequence[int],
            sampling_rows: Optional[dict] = None, drafts_dev: Optional[torch.Tensor] = None,
            state_slots: Optional[Sequence[int]] = None):
        """rows[i]: block-table row; tokens[i]: [pending, d_1 .. d_k]; starts[i]: position of the pending token;
        slot_lists[i]: the k + 1 reserved KV slots; sampling_rows: per-request lists temp / top_k / top_p / seed /
        draws / soft (all greedy when None); drafts_dev: int64 [n, k] drafts still on the device (tokens[i] then
        only needs its pending token; the drafted ids are copied into the static buffer on the stream, so the
        host never waits for them). Returns (emitted [n][k + 1], count [n], accepted [n], hidden)
        with the three lists on the host and `hidden` [bucket * (k + 1), H] on the device."""
        n, k1 = len(rows), self.k1
        self.runner._enter_forward()
        buf = self.bufs[self._bucket(n)]
        self._prepare(buf)
        tn, sn = buf.tok_np, buf.seq_np
        tn[:] = 0
        sn[:] = 0
        sn[S_CTX] = k1
        sn[S_BUDGET] = 1
        sn[S_STOP0:] = -1
        tn[T_POS] = np.tile(np.arange(k1, dtype=np.int32), buf.bucket)
        m = n * k1
        if drafts_dev is None:
            tn[T_IDS, :m] = np.asarray(tokens, dtype=np.int32).reshape(-1)
        else:
            tn[T_IDS, :m:k1] = [t[0] for t in tokens]
        st = np.asarray(starts, dtype=np.int32)
        tn[T_POS, :m] = (st[:, None] + np.arange(k1, dtype=np.int32)[None, :]).reshape(-1)
        tn[T_SLOT, :m] = np.asarray(slot_lists, dtype=np.int32).reshape(-1)
        tn[T_ROW, :m] = np.repeat(np.asarray(rows, dtype=np.int32), k1)
        sn[S_ROW, :n] = rows
        sn[S_CTX, :n] = st + k1
        sn[S_BUDGET, :n] = budgets
        if state_slots is not None:                         # padded requests keep the dummy slot 0
            sn[S_STATE, :n] = state_slots
        for i, ids in enumerate(stop_lists):
            ids = list(ids)[:MAX_STOPS]
            sn[S_STOP0:S_STOP0 + len(ids), i] = ids
        sn[S_TOPP].view(np.float32)[:] = 1.0
        if sampling_rows is not None:                       # rows left at zero are greedy (temperature 0)
            sn[S_TEMP].view(np.float32)[:n] = sampling_rows["temp"]
            sn[S_TOPK, :n] = sampling_rows["top_k"]
            sn[S_TOPP].view(np.float32)[:n] = sampling_rows["top_p"]
            sn[S_SOFT].view(np.float32)[:n] = sampling_rows["soft"]
            sn[S_SEED:S_SEED + 2].reshape(-1).view(np.int64)[:n] = sampling_rows["seed"]
            sn[S_DRAWS:S_DRAWS + 2].reshape(-1).view(np.int64)[:n] = sampling_rows["draws"]
        buf.dev.copy_(buf.host, non_blocking=True)
        self.runner.h2d_bytes += buf.host.numel() * 4
        if drafts_dev is not None:
            buf.tok[T_IDS].view(buf.bucket, k1)[:n, 1:].copy_(drafts_dev)
        if buf.graph is not None:
            buf.graph.replay()
        else:
            self._prepare(buf)
            self._body(buf)
        buf.meta_host.copy_(buf.meta, non_blocking=True)
        self.runner._queue_status_read()
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.runner.d2h_bytes += buf.meta.numel() * 8
        self.runner._raise_on_status()
        self.rounds += 1
        meta = buf.meta_host[:n].tolist()
        return ([row[:k1] for row in meta], [row[k1] for row in meta], [row[k1 + 1] for row in meta], buf.hidden)


D_IDS, D_POS, D_ROW, D_SLOT0 = 0, 1, 2, 3        # rows of the draft graphs' int32 buffer (k slot rows follow)


class DraftBuffers:
    def __init__(self, bucket: int, k: int, hidden: int, device: torch.device):
        self.bucket = bucket
        pin = device.type == "cuda"
        self.host = torch.zeros(D_SLOT0 + k, bucket, dtype=torch.int32, pin_memory=pin)
        self.np = self.host.numpy()
        self.dev = torch.zeros(D_SLOT0 + k, bucket, dtype=torch.int32, device=device)
        self.feat = torch.zeros(bucket, hidden, dtype=torch.bfloat16, device=device)
        self.drafts = torch.zeros(bucket, k, dtype=torch.int64, device=device)
        self.indptr = torch.arange(bucket + 1, dtype=torch.int32, device=device)
        self.graph = None


class DraftGraphs:
    """The MTP head's k chained draft steps (embed + fuse with the previous hidden, attention over the head's own
    KV, MLP, shared lm_head, argmax; the token feeds the next step) as one captured graph per batch bucket. The
    drafted ids stay on the device: the verify graph reads them there, so a speculative round is two pinned
    uploads, two graph replays and one read-back. Reference: hibana/proposers/mtp_graphs.py:15-120."""

    def __init__(self, runner, mtp, depth: int, buckets: Optional[Sequence[int]] = None):
        self.runner, self.model, self.mtp, self.k = runner, runner.model, mtp, depth
        self.device = runner.device
        self.buckets = tuple(buckets or runner.buckets)
        hidden = self.model.target.hidden
        self.bufs = {b: DraftBuffers(b, depth, hidden, self.device) for b in self.buckets}
        self.launches: dict = {}
        self.rounds = 0

    def _body(self, buf: DraftBuffers) -> None:
        r, b = self.runner, buf.bucket
        d = buf.dev
        hid, ids = buf.feat, d[D_IDS].long()
        for j in range(self.k):
            pos = d[D_POS] + j
            ctx = ForwardContext(VERIFY, positions=pos, slots=d[D_SLOT0 + j], kv_indices=r.block_table,
                                 ctx_len=pos + 1, q_indptr=buf.indptr, seq_rows=d[D_ROW], max_rows=1, batch=b,
                                 comm=r.comm, seq_starts_host=[1] * b)
            hid, normed = self.mtp.forward(hid, ids, ctx, r.kv)
            logits = self.model.logits(normed, r.comm) if r.comm is not None else self.model.logits(normed)
            ids = sampling.argmax(logits)
            buf.drafts[:, j].copy_(ids)

    def capture(self) -> None:
        if self.device.type != "cuda" or not self.runner.use_graphs:
            return
        for buf in self.bufs.values():
            buf.dev.zero_()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._body(buf)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = nv.LAUNCHES
            with torch.cuda.graph(g):
                self._body(buf)
            self.launches[buf.bucket] = nv.LAUNCHES - before
            buf.graph = g

    def run(self, rows: Sequence[int], pending: Sequence[int], positions: Sequence[int],
            slot_lists: Sequence[Sequence[int]], feat: torch.Tensor) -> torch.Tensor:
        """rows[i]: block-table row; pending[i]: the token whose successor is drafted first; positions[i]: the
        position of the hidden state `feat[i]` (the pending token sits one further); slot_lists[i]: the head's k KV
        slots from there. Returns the drafts int64 [n, k], on the device."""
        n = len(rows)
        buf = None
        for b in self.buckets:
            if b >= n:
                buf = self.bufs[b]
                break
        if buf is None:
            raise ValueError(f"batch {n} exceeds the largest draft bucket {self.buckets[-1]}")
        a = buf.np
        a[:] = 0
        a[D_IDS, :n] = pending
        a[D_POS, :n] = positions
        a[D_ROW, :n] = rows
        a[D_SLOT0:, :n] = np.asarray(slot_lists, dtype=np.int32).T
        buf.dev.copy_(buf.host, non_blocking=True)
        buf.feat[:n].copy_(feat)
        self.runner.h2d_bytes += buf.host.numel() * 4
        if buf.graph is not None:
            buf.graph.replay()
        else:
            self._body(buf)
        self.rounds += 1
        return buf.drafts[:n]
