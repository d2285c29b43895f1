"""Speculative decoding: draft with the MTP head, verify with the target, accept, commit.

A round for requests whose pending token x_n sits at position n (KV committed for 0..n-1):
  1. reserve k + 1 KV slots (positions n..n+k) as one transaction;
  2. draft: k chained MTP steps. Step 1 consumes (target hidden of position n-1, x_n) at MTP position n-1, step j
     consumes (previous draft hidden, d_{j-1}) at position n+j-2; the MTP layer keeps its KV in an extra layer of the
     same pool slots, so prefix-cache hits share it;
  3. verify: one ragged target forward over rows [x_n, d_1..d_k]; recurrent layers write to a scratch state slot and
     log their recurrence inputs;
  4. accept: longest prefix with d_{j+1} == target_j plus the target's own token (device kernel), truncated at stop
     ids and the token budget. Two other rules reuse that kernel by rewriting the "target" row it compares with:
     relaxed greedy (`accept_top_k` / `accept_margin`: a draft within the target's top-K and within the margin of
     the argmax counts as a match) and sampled acceptance for non-greedy requests (speculative sampling with the
     MTP argmax as a one-hot draft law: accept with probability p[d], else draw from p without d; engine/rejection.py);
  5. commit: keep the accepted slots, replay exactly the accepted rows of every recurrent layer from the untouched
     committed state (same kernels, so the state is bitwise what a plain decode would have produced), refresh the MTP
     KV of accepted positions with the true target hiddens.
Reference: hibana/engine/spec.py:268-741, hibana/proposers/mtp.py:187-376, hibana/engine/accept.py:18-56.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..utils import nvtx
from ..ops import sampling
from .context import DECODE, VERIFY, ForwardContext
from .request import MAX_STOPS, Request


class SpecStats:
    def __init__(self):
        self.rounds = self.proposed = self.accepted = self.emitted = 0

    def as_dict(self) -> dict:
        r = max(self.rounds, 1)
        return {"rounds": self.rounds, "proposed": self.proposed, "accepted": self.accepted, "emitted": self.emitted,
                "accept_rate": self.accepted / max(self.proposed, 1), "tokens_per_round": self.emitted / r}


class SpecDecoder:
    def __init__(self, executor, depth: int = 2, proposer=None):
        self.ex = executor
        self.model = executor.model
        self.mtp = getattr(executor.model, "mtp", None)
        # `proposer` (engine/contracts.py Proposer: n-gram lookup, block drafter, ...) replaces the built-in MTP
        # drafting; verification, acceptance and state replay are the same for every source of drafts
        self.proposer = proposer
        assert self.mtp is not None or proposer is not None, "speculation needs an MTP head or a proposer"
        self._started: set = set()
        self._laws = None
        self.depth = depth
        self.stats = SpecStats()
        self.feats: dict[int, torch.Tensor] = {}          # rid -> target hidden of the last committed position
        self.scratch: dict[int, int] = {}                 # rid -> scratch state slot (recurrent models)
        # captured verify + device accept (engine/spec_graphs.py): exact greedy rounds of unconstrained requests
        from .. import config as cfgmod
        from .spec_graphs import VerifyGraphs
        self.graphs = VerifyGraphs(executor.runner, depth) if cfgmod.current().device_accept else None
        if self.graphs is not None and not self.graphs.supported():
            self.graphs = None
        # the MTP head's chained draft steps as one graph per bucket; its drafts feed the verify graph on the device
        self.draft_graphs = None
        if self.graphs is not None and self.mtp is not None and proposer is None:
            from .spec_graphs import DraftGraphs
            self.draft_graphs = DraftGraphs(executor.runner, self.mtp, depth)

    # ---- helpers
    def _dev(self, arr, dtype):
        return torch.as_tensor(np.asarray(arr), dtype=dtype).to(self.ex.device)

    def _mtp_rows(self, reqs: Sequence[Request], hiddens: torch.Tensor, next_ids, positions, counts):
        """One MTP forward over ragged rows; returns (chained hidden, argmax token of every row)."""
        runner = self.ex.runner
        dev = self.ex.device
        b = len(reqs)
        counts = list(counts)
        indptr = np.zeros(b + 1, dtype=np.int32)
        indptr[1:] = np.cumsum(counts)
        pos = np.asarray(positions, dtype=np.int32)
        slots = np.concatenate([np.asarray(r.kv_slots[p0:p0 + c], dtype=np.int32)
                                for r, p0, c in zip(reqs, self._starts(pos, indptr), counts)])
        ctx_len = np.asarray([int(pos[indptr[i + 1] - 1]) + 1 for i in range(b)], dtype=np.int32)
        ctx = ForwardContext(VERIFY, positions=self._dev(pos, torch.int32), slots=self._dev(slots, torch.int32),
                             kv_indices=runner.block_table, ctx_len=self._dev(ctx_len, torch.int32),
                             q_indptr=self._dev(indptr, torch.int32),
                             seq_rows=self._dev([r.table_row for r in reqs], torch.int32), max_rows=max(counts),
                             batch=b)
        ids_t = next_ids if isinstance(next_ids, torch.Tensor) else self._dev(next_ids, torch.int64)
        g, normed = self.mtp.forward(hiddens, ids_t, ctx, self.ex.kv)
        tok = sampling.argmax(self.model.logits(normed))
        return g, tok

    def _decide(self, reqs: Sequence[Request], logits: torch.Tensor, drafts: torch.Tensor,
                bitmask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Per request, the token row the exact-match kernel compares the drafts with: the target argmax (exact
        greedy), the drafts themselves where the relaxed rule accepts them, or the outcome of speculative
        sampling. Nothing leaves the device."""
        from . import rejection
        b, k1, v = logits.shape
        k = k1 - 1
        dev = logits.device
        flat = logits.reshape(b * k1, v)
        out = sampling.argmax(flat, bitmask).view(b, k1).clone()      # grammar rows: argmax over the allowed tokens
        if bitmask is not None:
            flat = sampling._apply_bitmask(flat, bitmask)               # the rules below see -inf for forbidden tokens
            logits = flat.view(b, k1, v)
        greedy = torch.tensor([r.params.greedy for r in reqs], device=dev)
        rel = torch.tensor([r.params.greedy and (r.params.accept_top_k > 1 or r.params.accept_margin > 0)
                            for r in reqs], device=dev)
        if bool(rel.any()) and k:
            rank, gap = sampling.rank_gap(logits[:, :k].reshape(b * k, v).contiguous(), drafts.reshape(-1))
            topk = torch.tensor([max(r.params.accept_top_k, 1) for r in reqs], device=dev)[:, None]
            margin = torch.tensor([r.params.accept_margin for r in reqs], device=dev)[:, None]
            ok = (rank.view(b, k) < topk) & ((gap.view(b, k) <= margin) | (rank.view(b, k) == 0)) & rel[:, None]
            out[:, :k] = torch.where(ok, drafts, out[:, :k])
        if not bool(greedy.all()) and self._laws is None and not bool(rel.any()):
            # deterministic drafts (MTP, n-gram): the whole rejection-sampling rule is one kernel over the logits;
            # greedy requests of the batch keep the argmax computed above
            def col(vals, dtype):
                return torch.tensor(vals, dtype=dtype).to(dev)
            target, _ = sampling.spec_targets(
                flat, drafts, col([r.params.temperature for r in reqs], torch.float32),
                col([r.params.top_k for r in reqs], torch.int32), col([r.params.top_p for r in reqs], torch.float32),
                col([r.seed & 0x7FFFFFFFFFFFFFFF for r in reqs], torch.int64), col([r.draws for r in reqs], torch.int64),
                col([r.params.accept_soft for r in reqs], torch.float32), bitmask, greedy_pick=out.view(-1))
            return target
        if not bool(greedy.all()):
            temp = torch.tensor([r.params.temperature for r in reqs], device=dev).repeat_interleave(k1)
            tk = torch.tensor([r.params.top_k for r in reqs], device=dev).repeat_interleave(k1)
            tp = torch.tensor([r.params.top_p for r in reqs], device=dev).repeat_interleave(k1)
            laws = rejection.distribution(flat, temp, tk, tp).view(b, k1, v)
            if self._laws is not None:                                   # the proposer sampled from these
                q = self._laws.view(b, k, v).float()
            else:
                q = torch.zeros(b, k, v, device=dev)
                q.scatter_(2, drafts[:, :, None], 1.0)                   # deterministic drafts: a point mass
            u = torch.empty(b, k1, 2)
            for i, r in enumerate(reqs):                                 # counter-based: replay-safe
                for j in range(k1):
                    u[i, j, 0] = sampling.uniform01(r.seed, 2 * (r.draws + j) + 1)
                    u[i, j, 1] = sampling.uniform01(r.seed, 2 * (r.draws + j) + 2)
            u = u.to(dev)
            ver = rejection.verify_batch(laws, q, drafts, u[..., 0].contiguous(), u[..., 1].contiguous(),
                                         soft=torch.tensor([r.params.accept_soft for r in reqs], device=dev))
            out = torch.where(greedy[:, None], out, ver.emitted)
        return out

    @staticmethod
    def _starts(pos, indptr):
        return [int(pos[indptr[i]]) for i in range(len(indptr) - 1)]

    # ---- prefill hook
    def ingest_prefill(self, req: Request, hidden: torch.Tensor, start: int, count: int) -> None:
        """After a target prefill chunk over positions [start, start + count): feed the MTP layer the pairs
        (h_p, x_{p+1}) whose next token is already known and keep the last hidden as the request's feature."""
        if self.proposer is not None:
            self.proposer.ingest_prefill(req, hidden, start, count)
            self.feats[req.rid] = hidden[count - 1].clone()
            return
        seq = req.all_ids
        rows, ids, pos = [], [], []
        prev = self.feats.get(req.rid)
        if start > 0:
            rows.append(prev if prev is not None else torch.zeros_like(hidden[0]))   # stand-in on a cache hit
            ids.append(seq[start])
            pos.append(start - 1)
        for j in range(count - 1):
            rows.append(hidden[j])
            ids.append(seq[start + j + 1])
            pos.append(start + j)
        self.feats[req.rid] = hidden[count - 1].clone()
        if rows:
            self._mtp_rows([req], torch.stack(rows), ids, pos, [len(rows)])

    def release(self, req: Request) -> None:
        self.feats.pop(req.rid, None)
        if self.proposer is not None:
            self._started.discard(req.rid)
            self.proposer.release(req)
        slot = self.scratch.pop(req.rid, None)
        if slot and self.ex.state_pool is not None:
            self.ex.state_pool.free(slot)

    # ---- the round
    @nvtx.ranged("spec_round")
    def round(self, reqs: Sequence[Request]) -> None:
        ex, dev = self.ex, self.ex.device
        k = self.depth
        b = len(reqs)
        ex.state.reserve(reqs, k + 1)                      # MemoryError -> the scheduler retracts and retries
        n = [r.total_len - 1 for r in reqs]                # position of the pending token
        for r, nn in zip(reqs, n):                         # the block table must know the reserved slots
            ex.runner.set_table(r.table_row, nn, r.kv_slots[nn:nn + k + 1])
        # ---- draft
        feat = torch.stack([self.feats.get(r.rid, torch.zeros(self.model.target.hidden, dtype=torch.bfloat16,
                                                              device=dev)) for r in reqs])
        drafts = torch.zeros(b, k, dtype=torch.int64, device=dev)
        self._laws = None
        if self.proposer is not None:
            for r in reqs:
                if r.rid not in self._started:
                    self._started.add(r.rid)
                    self.proposer.start(r)
            prop = self.proposer.propose(reqs, k)
            toks = prop if isinstance(prop, torch.Tensor) else prop.tokens
            drafts.copy_(toks.view(b, k))           # short drafts arrive padded: a padded token is simply refused
            if not isinstance(prop, torch.Tensor) and prop.laws is not None:
                self._laws = prop.laws.to(dev)
        elif self.draft_graphs is not None and b <= self.draft_graphs.buckets[-1]:
            drafts = self.draft_graphs.run([r.table_row for r in reqs], [r.output_ids[-1] for r in reqs],
                                           [nn - 1 for nn in n], [r.kv_slots[nn - 1:nn - 1 + k] for r, nn in zip(reqs, n)],
                                           feat)
        else:
            hid = feat
            ids = [r.output_ids[-1] for r in reqs]
            for j in range(k):
                hid, tok = self._mtp_rows(reqs, hid, ids, [nn - 1 + j for nn in n], [1] * b)
                drafts[:, j] = tok
                ids = tok if j + 1 < k else None
        # ---- verify
        on_device = (self.draft_graphs is not None and self.proposer is None and self.graphs is not None
                     and b <= self.graphs.buckets[-1]
                     and not any(r.grammar is not None for r in reqs)
                     and not any(r.params.greedy and (r.params.accept_top_k > 1 or r.params.accept_margin > 0)
                                 for r in reqs))
        host_drafts = [[0] * k for _ in reqs] if on_device else drafts.tolist()   # on_device: no wait for the drafts
        tokens = [[r.output_ids[-1]] + host_drafts[i] for i, r in enumerate(reqs)]
        extras = {"want_hidden": True}
        has_state = ex.state_pool is not None
        relaxed = any(r.params.greedy and (r.params.accept_top_k > 1 or r.params.accept_margin > 0) for r in reqs)
        sampled = any(not r.params.greedy for r in reqs)
        # grammar-constrained requests: the drafted tokens are walked through the grammar on the host, one mask per
        # verified row (the state after the drafted prefix before it); acceptance then runs on the masked logits,
        # so a drafted token the grammar forbids can never be accepted and the correction comes from a masked row
        bitmask = None
        if any(r.grammar is not None for r in reqs):
            from .grammar import stack_masks
            rows_m = []
            for i, r in enumerate(reqs):
                rows_m.extend(r.grammar.verify_masks(host_drafts[i]) if r.grammar is not None else [None] * (k + 1))
            bitmask = stack_masks(rows_m, (self.model.target.vocab + 31) // 32)
            if bitmask is not None:
                bitmask = bitmask.to(dev)
        stop_lists = []
        for r in reqs:
            ids_ = list(r.params.stop_ids)[:MAX_STOPS]
            if r.eos_id is not None and not r.params.ignore_eos and len(ids_) < MAX_STOPS:
                ids_.append(r.eos_id)
            stop_lists.append(ids_)
        budgets = [max(r.remaining, 1) for r in reqs]
        slot_lists = [r.kv_slots[nn:nn + k + 1] for r, nn in zip(reqs, n)]
        in_graph = (self.graphs is not None and not (relaxed or bitmask is not None)
                    and (not sampled or self._laws is None) and b <= self.graphs.buckets[-1])
        if has_state and not in_graph:
            for r in reqs:
                if r.rid not in self.scratch:
                    self.scratch[r.rid] = ex.state_pool.alloc()
            extras["state_out"] = self._dev([self.scratch[r.rid] for r in reqs], torch.int32)
            extras["ring"] = []
        if in_graph:
            # one upload, one captured verify + accept, one readback (engine/spec_graphs.py)
            srows = None
            if sampled:
                srows = {"temp": [r.params.temperature for r in reqs], "top_k": [r.params.top_k for r in reqs],
                         "top_p": [r.params.top_p for r in reqs], "soft": [r.params.accept_soft for r in reqs],
                         "seed": [r.seed & 0x7FFFFFFFFFFFFFFF for r in reqs], "draws": [r.draws for r in reqs]}
            emitted_h, count_h, acc_h, hidden = self.graphs.run([r.table_row for r in reqs], tokens, n, slot_lists,
                                                                stop_lists, budgets, srows,
                                                                drafts_dev=drafts if on_device else None,
                                                                state_slots=[r.state_slot for r in reqs]
                                                                if has_state else None)
        else:
            target, hidden = ex.runner.forward_rows(
                [r.table_row for r in reqs], tokens, n, slot_lists, mode=VERIFY,
                want="logits_device" if (relaxed or sampled or bitmask is not None) else "all_device",
                state_slots=[r.state_slot for r in reqs] if has_state else None, extras=extras)
            if relaxed or sampled or bitmask is not None:
                target = self._decide(reqs, target.view(b, k + 1, -1), drafts, bitmask)
            target = target.view(b, k + 1)
            # ---- accept (device), one small readback
            stops = torch.full((b, MAX_STOPS), -1, dtype=torch.int64)
            for i, ids_ in enumerate(stop_lists):
                stops[i, :len(ids_)] = torch.tensor(ids_, dtype=torch.int64) if ids_ else stops[i, :0]
            budget = torch.tensor(budgets, dtype=torch.int32)
            emitted, count, accepted = sampling.accept_greedy(target, drafts, stops.to(dev), budget.to(dev))
            emitted_h, count_h, acc_h = emitted.tolist(), count.tolist(), accepted.tolist()
        # ---- commit
        sel_rows, new_indptr = [], [0]
        for i, r in enumerate(reqs):
            c = count_h[i]
            ex.state.commit(r, c)
            sel_rows.extend(range(i * (k + 1), i * (k + 1) + c))
            new_indptr.append(new_indptr[-1] + c)
            self.feats[r.rid] = hidden[i * (k + 1) + c - 1].clone()
        if has_state and not in_graph:              # (a captured round replayed the accepted rows itself)
            sel = self._dev(sel_rows, torch.int64)
            ip = self._dev(new_indptr, torch.int32)
            slots = self._dev([r.state_slot for r in reqs], torch.int32)
            for layer, saved in extras["ring"]:
                layer.replay(saved, sel, ip, slots, ex.state_pool)
        if self.proposer is not None:
            from .contracts import VerifiedFeatures
            self.proposer.accepted_batch(reqs, [emitted_h[i][:count_h[i]] for i in range(b)],
                                         VerifiedFeatures(hidden, count_h, k + 1))
        # refresh the MTP KV of accepted draft positions with the true target hiddens
        ref_reqs, ref_rows, ref_ids, ref_pos, ref_cnt = [], [], [], [], []
        for i, r in enumerate(reqs if self.proposer is None else []):
            a = count_h[i] - 1
            if a > 0:
                ref_reqs.append(r)
                ref_rows.extend(range(i * (k + 1), i * (k + 1) + a))
                ref_ids.extend(emitted_h[i][:a])
                ref_pos.extend(range(n[i], n[i] + a))
                ref_cnt.append(a)
        if ref_reqs:
            self._mtp_rows(ref_reqs, hidden.index_select(0, self._dev(ref_rows, torch.int64)), ref_ids, ref_pos,
                           ref_cnt)
        for i, r in enumerate(reqs):
            c = count_h[i]
            r.draws += c
            r.rounds.append(c)
            for tok in emitted_h[i][:c]:
                if r.push(tok):
                    break
            self.stats.rounds += 1
            self.stats.proposed += k
            self.stats.accepted += acc_h[i]
            self.stats.emitted += c
