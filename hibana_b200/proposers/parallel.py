"""Block ("parallel") drafting proposer: one drafter forward drafts the whole verify block.

Per request the proposer keeps a ring of the drafter's context entries (keys / values per drafter layer for the last
`window` committed tokens, computed from the token and the target's hidden state at that position; see
models/parallel_draft.py). It never touches target KV or state: `ingest_prefill` appends entries for prompt
chunks, `accepted_batch` for the tokens a round committed (with the target hiddens of the verified rows), `propose`
runs the block forward over [anchor, mask x depth] for all requests at once and walks the candidate lattice:
greedy for greedy requests, sampled (with the law of every draw, for speculative sampling) otherwise.
Reference: hibana/proposers/parallel.py:60-277 (state ring, propose, feedback), MAX_DEPTHS["dflash2"] = 15.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..engine.contracts import Capabilities, Proposal, VerifiedFeatures
from ..models.parallel_draft import BlockDrafter
from ..ops.sampling import lattice_walk
from ..ops.sampling import uniform01


class _Ring:
    def __init__(self, layers: int, window: int, heads: int, hd: int, device, dtype):
        self.k = torch.zeros(layers, window, heads, hd, device=device, dtype=dtype)
        self.v = torch.zeros(layers, window, heads, hd, device=device, dtype=dtype)
        self.end = 0            # committed tokens seen (entries live at position % window)
        self.first = 0          # earliest position held (a cache hit may start the ring late)


class ParallelProposer:
    capabilities = Capabilities(short_drafts=False, scored_drafts=True, max_depth=15)

    def __init__(self, drafter: BlockDrafter):
        self.m = drafter
        self.rings: dict[int, _Ring] = {}

    # ---- context ring
    def _ring(self, req) -> _Ring:
        r = self.rings.get(req.rid)
        if r is None:
            m = self.m
            r = self.rings[req.rid] = _Ring(m.nl, m.window, m.nh, m.hd, m.device, m.dtype)
        return r

    def _append(self, req, tokens: Sequence[int], hidden: torch.Tensor, start: int) -> None:
        n = len(tokens)
        if n == 0:
            return
        ring, m = self._ring(req), self.m
        if n > m.window:                              # only the tail can survive in the ring
            tokens, hidden, start, n = tokens[-m.window:], hidden[-m.window:], start + n - m.window, m.window
        if ring.end != start:                         # a gap (prefix served from the cache): restart the ring here
            ring.first = start
        pos = torch.arange(start, start + n, device=m.device)
        kv = m.context_kv(torch.as_tensor(list(tokens), device=m.device), hidden.to(m.device), pos)
        idx = pos % m.window
        for li, (k, v) in enumerate(kv):
            ring.k[li, idx] = k
            ring.v[li, idx] = v
        ring.end = start + n
        ring.first = max(ring.first, ring.end - m.window)

    def ingest_prefill(self, req, hidden: torch.Tensor, start: int, count: int) -> None:
        self._append(req, req.all_ids[start:start + count], hidden[:count], start)

    def start(self, req) -> None:
        self._ring(req)

    def ready(self, reqs: Sequence) -> bool:
        return True

    # ---- drafting
    def propose(self, reqs: Sequence, depth: int) -> Proposal:
        m = self.m
        b = len(reqs)
        dev = m.device
        anchors = torch.tensor([r.output_ids[-1] if r.output_ids else r.prompt_ids[-1] for r in reqs], device=dev)
        positions = torch.tensor([r.total_len - 1 for r in reqs], device=dev)
        ck = torch.stack([self._ring(r).k for r in reqs], 1)        # [layers, B, window, heads, d]
        cv = torch.stack([self._ring(r).v for r in reqs], 1)
        mask = torch.zeros(b, m.window, dtype=torch.bool, device=dev)
        for i, r in enumerate(reqs):                                # position p lives in slot p % window
            ring = self._ring(r)
            held = ring.end - ring.first
            if held > 0:
                live = torch.arange(ring.first, ring.end, device=dev) % m.window
                mask[i, live] = True
        hidden = m.forward(anchors, positions, list(ck), list(cv), mask, depth)
        cand, scores = m.select(hidden, anchors)
        greedy = all(r.params.greedy for r in reqs)
        temp = u = None
        if not greedy:
            temp = torch.tensor([0.0 if r.params.greedy else max(r.params.temperature, 1e-6) for r in reqs],
                                dtype=torch.float32, device=dev)
            u = torch.tensor([[uniform01(r.seed ^ 0x5DEECE66D, r.draws + j) for j in range(depth)] for r in reqs],
                             dtype=torch.float32, device=dev)
        # one warp per request walks the lattice (ops/sampling.py `lattice_walk`): tokens, the law each was drawn
        # from on its candidates, and the acceptance estimate (unit-temperature mass of the choice) in one launch
        toks, idx, probs, est = lattice_walk(cand, scores, temp, u)
        laws = None
        if not greedy:       # speculative sampling wants the draft law dense over the vocabulary
            laws = torch.zeros(b, depth, m.vocab, device=dev)
            laws.scatter_add_(2, cand, probs)
        return Proposal(toks, laws=laws, scores=est)

    # ---- feedback
    def accepted_batch(self, reqs: Sequence, emitted: Sequence[Sequence[int]],
                       features: Optional[VerifiedFeatures]) -> None:
        if features is None:
            return
        rpr = features.rows_per_request
        for i, r in enumerate(reqs):
            c = int(features.counts[i])
            if c <= 0:
                continue
            # the rows verified were [pending token, drafts...]; the first c of them are now committed: the pending
            # token (still the last id of the request: this runs before the emitted tokens are pushed) and the
            # first c - 1 emitted ones. The c-th emitted token is the next round's pending token.
            start = r.total_len - 1
            toks = [r.all_ids[-1]] + [int(t) for t in emitted[i][:c - 1]]
            self._append(r, toks, features.hidden[i * rpr:i * rpr + c], start)

    def release(self, req) -> None:
        self.rings.pop(req.rid, None)
