"""How many tokens to draft: fixed, per batch bucket, adapted per request from an acceptance estimate, or chosen
after drafting under a budget of verify rows.

  FixedDepth(k)                 the same depth for everyone
  BatchDepth("1:6,8:4,32:2")    depth by batch size (largest threshold <= batch wins); 0 = plain decode
  AcceptanceDepth               per request: an exponential moving average a of the per-position acceptance rate
                                (alpha 0.1, prior 0.8) gives the expected tokens of depth k, sum_{j<=k} a^j; the
                                depth is the largest k whose marginal gain a^k still pays for a verify row
  RowBudget                     after drafting: given each request's draft scores (estimated acceptance of every
                                drafted position), keep the globally most promising rows until the verify-row
                                budget of the step is spent (ragged verify)
Reference: hibana/engine/depth.py:23-331, docs/interfaces.md:124-138.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


class FixedDepth:
    def __init__(self, depth: int):
        self.depth = depth

    def depths(self, reqs: Sequence) -> list[int]:
        return [self.depth] * len(reqs)

    def observe(self, req, proposed: int, accepted: int) -> None:
        pass


def parse_depths(spec: str) -> list[tuple[int, int]]:
    """'1:6,8:4,32:2' -> [(1, 6), (8, 4), (32, 2)] sorted by batch threshold."""
    out = []
    for part in spec.split(","):
        part = part.strip()
        if not part:
            continue
        a, _, b = part.partition(":")
        if not _:
            raise ValueError(f"depth table entry '{part}' is not batch:depth")
        out.append((int(a), int(b)))
    if not out:
        raise ValueError("empty depth table")
    if any(bt < 1 or d < 0 for bt, d in out):
        raise ValueError("depth table needs batch >= 1 and depth >= 0")
    return sorted(out)


class BatchDepth:
    def __init__(self, table: str | Sequence[tuple[int, int]]):
        self.table = parse_depths(table) if isinstance(table, str) else sorted(table)

    def depth_for(self, batch: int) -> int:
        d = self.table[0][1]
        for threshold, depth in self.table:
            if batch >= threshold:
                d = depth
        return d

    def depths(self, reqs: Sequence) -> list[int]:
        return [self.depth_for(len(reqs))] * len(reqs)

    def observe(self, req, proposed: int, accepted: int) -> None:
        pass


class AcceptanceDepth:
    """Per-request adaptive depth. `row_cost` is the price of one more verify row in units of an emitted token
    (verify time per row / step time): drafting deeper pays while a^k > row_cost."""

    def __init__(self, max_depth: int = 8, alpha: float = 0.1, prior: float = 0.8, row_cost: float = 0.12,
                 min_depth: int = 1):
        self.max_depth, self.alpha, self.prior, self.row_cost, self.min_depth = max_depth, alpha, prior, row_cost, min_depth
        self.rate: dict[int, float] = {}

    def estimate(self, req) -> float:
        return self.rate.get(req.rid, self.prior)

    def depth_for(self, req) -> int:
        a = self.estimate(req)
        k, gain = 0, a
        while k < self.max_depth and gain > self.row_cost:
            k += 1
            gain *= a
        return max(k, self.min_depth)

    def depths(self, reqs: Sequence) -> list[int]:
        return [self.depth_for(r) for r in reqs]

    def observe(self, req, proposed: int, accepted: int) -> None:
        """Each drafted position up to and including the first rejection is one Bernoulli observation."""
        if proposed <= 0:
            return
        a = self.estimate(req)
        for j in range(min(accepted + 1, proposed)):
            a += self.alpha * ((1.0 if j < accepted else 0.0) - a)
        self.rate[req.rid] = min(max(a, 0.02), 0.995)

    def forget(self, req) -> None:
        self.rate.pop(req.rid, None)


def expected_tokens(rate: float, depth: int) -> float:
    """1 (the target's own token) + expected accepted drafts at per-position acceptance `rate`."""
    return 1.0 + sum(rate ** j for j in range(1, depth + 1))


@dataclass
class RowBudget:
    """Post-draft row budgeting: position j of request i is worth the probability that all of its first j drafts
    are accepted (the product of their scores); rows are kept in decreasing worth, a request's rows as a prefix."""
    rows: int                                  # verify rows per step (including each request's pending row)
    min_depth: int = 0
    kept: list = field(default_factory=list)

    def choose(self, scores: Sequence[Sequence[float]]) -> list[int]:
        n = len(scores)
        budget = self.rows - n                 # every request verifies its pending token
        depth = [min(self.min_depth, len(s)) for s in scores]
        budget -= sum(depth)
        worth = []
        for i, s in enumerate(scores):
            acc = 1.0
            for j, v in enumerate(s):
                acc *= min(max(float(v), 0.0), 1.0)
                if j >= depth[i]:
                    worth.append((acc, -j, i))
        worth.sort(reverse=True)
        for w, negj, i in worth:
            if budget <= 0:
                break
            if -negj == depth[i]:              # prefix property: only the next position of a request may be added
                depth[i] += 1
                budget -= 1
        # a second pass picks up positions skipped while their predecessor was still waiting
        changed = True
        while budget > 0 and changed:
            changed = False
            for w, negj, i in worth:
                if budget > 0 and -negj == depth[i]:
                    depth[i] += 1
                    budget -= 1
                    changed = True
        self.kept = depth
        return depth


def ragged_budgets(batch: int, rows: int, max_depth: int) -> int:
    """Verify rows a packed (ragged) verify graph of `rows` rows leaves per request on average."""
    return max(0, min(max_depth, rows // max(batch, 1) - 1))
