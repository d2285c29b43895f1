"""Prompt-lookup proposer: drafts the continuation that followed the longest recent n-gram match in the request's
own token history. No model, no device work; useful for copy-heavy workloads (code edits, retrieval answers) and as
the always-available fallback when no drafter head is loaded. Scores fall with the distance from the match.
(The reference's model-free fallback is plain decode; its DFlash2 block drafter needs trained weights.)"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..engine.contracts import Capabilities, Proposal, VerifiedFeatures


class NgramProposer:
    capabilities = Capabilities(short_drafts=True, scored_drafts=True, max_depth=15)

    def __init__(self, max_ngram: int = 4, min_ngram: int = 2, pad_token: int = 0):
        self.max_ngram, self.min_ngram, self.pad = max_ngram, min_ngram, pad_token

    def ingest_prefill(self, req, hidden, start, count) -> None:
        pass

    def start(self, req) -> None:
        pass

    def ready(self, reqs: Sequence) -> bool:
        return True

    def _lookup(self, seq: Sequence[int], depth: int) -> list[int]:
        n = len(seq)
        for size in range(min(self.max_ngram, n - 1), self.min_ngram - 1, -1):
            tail = seq[n - size:]
            for i in range(n - size - 1, -1, -1):          # latest earlier occurrence wins
                if seq[i:i + size] == tail:
                    return list(seq[i + size:i + size + depth])
        return []

    def propose(self, reqs: Sequence, depth: int) -> Proposal:
        toks, lens = [], []
        for r in reqs:
            d = self._lookup(r.all_ids, depth)
            lens.append(len(d))
            toks.append(d + [self.pad] * (depth - len(d)))
        scores = torch.tensor([[0.6 * (0.85 ** j) if j < n else 0.0 for j in range(depth)] for n in lens])
        return Proposal(torch.tensor(toks, dtype=torch.int64).view(len(reqs), depth), scores=scores, lengths=lens)

    def accepted_batch(self, reqs, emitted, features: Optional[VerifiedFeatures]) -> None:
        pass

    def release(self, req) -> None:
        pass
