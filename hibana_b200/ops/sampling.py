"""Sampling and speculative-acceptance ops (csrc/sample.cu) with plain-PyTorch references.

Reference counterparts: hibana/engine/sampler.py:87-123, hibana/engine/accept.py:18-56,
hibana/kernels/relaxed_rank.py:13.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native as nv

P, I, L = nv.P, nv.I, nv.L
nv.register("hb_argmax", [P, L, I, I, I, P, I, P, P, P])
nv.register("hb_sample", [P, L, I, I, I, P, P, P, P, P, P, I, P, P, I, P])
nv.register("hb_argmax2", [P, L, I, I, I, P, I, I, P, P, P, P, P, P])

ARGMAX_CHUNKS = 32
nv.register("hb_accept_greedy", [P, P, P, I, P, P, I, I, P, P, P, P])
nv.register("hb_rank_gap", [P, L, I, I, I, P, P, P, P])
nv.register("hb_lattice_walk", [P, P, P, P, I, I, I, P, P, P, P, P])
nv.register("hb_spec_targets", [P, L, I, I, I, I, P, P, P, P, P, P, P, P, I, P, P, P, P])

MASK64 = (1 << 64) - 1


def _apply_bitmask(logits: torch.Tensor, bitmask: Optional[torch.Tensor]) -> torch.Tensor:
    if bitmask is None:
        return logits.float()
    vocab = logits.shape[1]
    idx = torch.arange(vocab, device=logits.device)
    allowed = ((bitmask[:, (idx >> 5).long()] >> (idx & 31)) & 1).bool()
    return logits.float().masked_fill(~allowed, float("-inf"))


def argmax(logits: torch.Tensor, bitmask: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row (int64). `bitmask` int32 [rows, ceil(vocab/32)] allows token i when bit i is set."""
    rows, vocab = logits.shape
    if nv.use_native(logits):
        out = torch.empty(rows, dtype=torch.int64, device=logits.device) if out is None else out
        _argmax2(logits, bitmask, None, out)
        return out
    res = _apply_bitmask(logits, bitmask).argmax(dim=-1)
    if out is not None:
        out.copy_(res)
        return out
    return res


def argmax_with_value(logits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(index int64 [rows], value fp32 [rows]) of every row's maximum (lowest index on ties): the per-shard half of
    a vocab-parallel greedy pick."""
    rows = logits.shape[0]
    if nv.use_native(logits):
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
        val = torch.empty(rows, dtype=torch.float32, device=logits.device)
        _argmax2(logits, None, None, out, val)
        return out, val
    val, idx = logits.float().max(dim=-1)
    return idx, val


def _argmax2(logits: torch.Tensor, bitmask: Optional[torch.Tensor], temperature: Optional[torch.Tensor],
             out: torch.Tensor, out_val: Optional[torch.Tensor] = None) -> None:
    rows, vocab = logits.shape
    nch = ARGMAX_CHUNKS if vocab >= 8192 else 1
    sv = torch.empty(rows, nch, dtype=torch.float32, device=logits.device)
    si = torch.empty(rows, nch, dtype=torch.int32, device=logits.device)
    nv.check(nv.lib().hb_argmax2(logits.data_ptr(), logits.stride(0), rows, vocab, int(logits.dtype == torch.float32),
                                 nv.ptr(bitmask), bitmask.shape[1] if bitmask is not None else 0, nch, sv.data_ptr(),
                                 si.data_ptr(), nv.ptr(temperature), out.data_ptr(), nv.ptr(out_val), nv.stream()),
             "hb_argmax2",
             launches=2)


def uniform01(seed: int, offset: int) -> float:
    """Host copy of the device counter RNG (splitmix64 finaliser) so tests can predict draws."""
    z = (seed + 0x9E3779B97F4A7C15 * (offset + 1)) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def sample_ref(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
               seeds: torch.Tensor, offsets: torch.Tensor, bitmask: Optional[torch.Tensor] = None,
               max_k: int = 64) -> torch.Tensor:
    lg = _apply_bitmask(logits, bitmask)
    rows = lg.shape[0]
    out = torch.zeros(rows, dtype=torch.int64)
    for r in range(rows):
        t = float(temperature[r])
        if t <= 0:
            out[r] = int(lg[r].argmax())
            continue
        k = int(top_k[r])
        if k <= 0 or k > max_k:
            # top-k off or wider than the kernel's candidate list: the full-vocabulary law (softmax, then nucleus),
            # drawn by inverse CDF in index order
            from ..engine.rejection import distribution
            law = distribution(lg[r:r + 1].cpu(), t, k if k > max_k else 0, float(top_p[r]))[0].double()
            u = uniform01(int(seeds[r]), int(offsets[r])) * float(law.sum())
            acc = torch.cumsum(law, 0)
            hit = (u < acc).nonzero()
            out[r] = int(hit[0]) if len(hit) else int((law > 0).nonzero()[-1])
            continue
        vals, idx = torch.sort(lg[r].cpu(), descending=True, stable=True)
        vals, idx = vals[:k], idx[:k]
        w = torch.exp((vals - vals[0]) / t)
        w[vals == float("-inf")] = 0
        cum = torch.cumsum(w / w.sum(), 0)
        p = float(top_p[r])
        keep = k
        if p < 1.0:
            over = (cum >= p).nonzero()
            keep = int(over[0]) + 1 if len(over) else k
        w = w[:keep]
        u = uniform01(int(seeds[r]), int(offsets[r])) * float(w.sum())
        acc = torch.cumsum(w, 0)
        pick = int((u < acc).nonzero()[0]) if bool((u < acc).any()) else keep - 1
        out[r] = int(idx[pick])
    return out.to(logits.device)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seeds: torch.Tensor, offsets: torch.Tensor, bitmask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Temperature / top-k / top-p sampling; temperature <= 0 is greedy. seeds/offsets are uint64-as-int64.
    1 <= top-k <= 64 draws from the k largest logits in candidate order; top-k <= 0 (off) or > 64 draws in index
    order from the law `engine.rejection.distribution` gives speculative verification (softmax over the whole
    vocabulary or its k largest tokens, then top-p)."""
    rows, vocab = logits.shape
    if nv.use_native(logits):
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
        _argmax2(logits, bitmask, temperature, out)      # greedy rows
        nv.check(nv.lib().hb_sample(logits.data_ptr(), logits.stride(0), rows, vocab,
                                    int(logits.dtype == torch.float32), temperature.data_ptr(), top_k.data_ptr(),
                                    top_p.data_ptr(), seeds.data_ptr(), offsets.data_ptr(), nv.ptr(bitmask),
                                    bitmask.shape[1] if bitmask is not None else 0, out.data_ptr(), None, 1,
                                    nv.stream()), "hb_sample")   # rows with temperature > 0
        return out
    return sample_ref(logits, temperature, top_k, top_p, seeds, offsets, bitmask)


def accept_greedy_ref(target: torch.Tensor, drafts: torch.Tensor, stop_ids: Optional[torch.Tensor],
                      budget: Optional[torch.Tensor], depth: Optional[torch.Tensor]):
    b, k1 = target.shape
    kmax = k1 - 1
    emitted = torch.zeros(b, k1, dtype=torch.int64)
    count = torch.zeros(b, dtype=torch.int32)
    accepted = torch.zeros(b, dtype=torch.int32)
    for i in range(b):
        k = min(int(depth[i]), kmax) if depth is not None else kmax
        lim = int(budget[i]) if budget is not None else k + 1
        n = acc = 0
        for j in range(k + 1):
            if n >= lim:
                break
            tok = int(target[i, j])
            emitted[i, n] = tok
            n += 1
            if stop_ids is not None and tok in stop_ids[i].tolist():
                if j < k and int(drafts[i, j]) == tok:
                    acc += 1
                break
            if j < k and int(drafts[i, j]) == tok:
                acc += 1
            else:
                break
        count[i], accepted[i] = n, acc
    return emitted, count, accepted


def accept_greedy(target: torch.Tensor, drafts: torch.Tensor, stop_ids: Optional[torch.Tensor] = None,
                  budget: Optional[torch.Tensor] = None, depth: Optional[torch.Tensor] = None):
    """target [B, k+1] (argmax of every verify row), drafts [B, k] -> (emitted [B, k+1], count [B], accepted [B])."""
    b, k1 = target.shape
    if nv.use_native(target):
        emitted = torch.zeros(b, k1, dtype=torch.int64, device=target.device)
        count = torch.empty(b, dtype=torch.int32, device=target.device)
        accepted = torch.empty(b, dtype=torch.int32, device=target.device)
        nv.check(nv.lib().hb_accept_greedy(target.data_ptr(), drafts.data_ptr(), nv.ptr(stop_ids),
                                           stop_ids.shape[1] if stop_ids is not None else 0, nv.ptr(budget),
                                           nv.ptr(depth), k1 - 1, b, emitted.data_ptr(), count.data_ptr(),
                                           accepted.data_ptr(), nv.stream()), "hb_accept_greedy")
        return emitted, count, accepted
    e, c, a = accept_greedy_ref(target.cpu(), drafts.cpu(), stop_ids, budget, depth)
    return e.to(target.device), c.to(target.device), a.to(target.device)


def rank_gap(logits: torch.Tensor, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Rank (count of strictly larger logits) and logit gap to the maximum of token ids[row] in its row."""
    rows, vocab = logits.shape
    if nv.use_native(logits):
        rank = torch.empty(rows, dtype=torch.int32, device=logits.device)
        gap = torch.empty(rows, dtype=torch.float32, device=logits.device)
        nv.check(nv.lib().hb_rank_gap(logits.data_ptr(), logits.stride(0), rows, vocab,
                                      int(logits.dtype == torch.float32), ids.data_ptr(), rank.data_ptr(),
                                      gap.data_ptr(), nv.stream()), "hb_rank_gap")
        return rank, gap
    lg = logits.float()
    mine = lg.gather(1, ids.view(-1, 1))
    return (lg > mine).sum(1).int(), (lg.max(1).values - mine.squeeze(1))


def spec_targets_ref(logits: torch.Tensor, drafts: torch.Tensor, temperature, top_k, top_p, seeds, draws, soft,
                     bitmask: Optional[torch.Tensor] = None):
    """Plain PyTorch `spec_targets` (same uniforms, same law, draws by inverse CDF in index order)."""
    from ..engine.rejection import distribution
    b, k = drafts.shape
    k1 = k + 1
    lg = _apply_bitmask(logits, bitmask).cpu().view(b, k1, -1)
    target = torch.zeros(b, k1, dtype=torch.int64)
    p_draft = torch.ones(b, k1, dtype=torch.float32)

    def draw(law, u):
        acc = torch.cumsum(law.double(), 0)
        hit = (u * float(acc[-1]) < acc).nonzero()
        return int(hit[0]) if len(hit) else int((law > 0).nonzero()[-1])
    for i in range(b):
        t = float(temperature[i])
        laws = distribution(lg[i], t, int(top_k[i]) if t > 0 else 1, float(top_p[i]) if t > 0 else 1.0)
        for j in range(k1):
            u_res = uniform01(int(seeds[i]), 2 * (int(draws[i]) + j) + 2)
            if j == k:
                target[i, j] = draw(laws[j], u_res)
                continue
            d = int(drafts[i, j])
            pd = float(laws[j, d])
            p_draft[i, j] = pd
            u = uniform01(int(seeds[i]), 2 * (int(draws[i]) + j) + 1)
            sf = float(soft[i]) if soft is not None else 0.0
            if u < pd or (sf > 0 and u < math.exp(sf) * pd):
                target[i, j] = d
                continue
            res = laws[j].clone()
            res[d] = 0
            target[i, j] = draw(res if float(res.sum()) > 1e-6 * float(laws[j].sum()) else laws[j], u_res)
    return target.to(logits.device), p_draft.to(logits.device)


def spec_targets(logits: torch.Tensor, drafts: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                 top_p: torch.Tensor, seeds: torch.Tensor, draws: torch.Tensor, soft: Optional[torch.Tensor] = None,
                 bitmask: Optional[torch.Tensor] = None,
                 greedy_pick: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Speculative rejection sampling against deterministic drafts in one kernel. logits [B * (k + 1), V] (request b
    owns rows b * (k + 1) ...), drafts int64 [B, k], per-request temperature / top_k / top_p / seeds / draws (the
    request's draw counter) / soft (relaxed acceptance, e^soft on the test). Returns (target int64 [B, k + 1],
    p_draft fp32 [B, k + 1]): target[b, j] is drafts[b, j] where the draft stands, the draw from the residual law
    where it does not, and the bonus draw at j = k, so `accept_greedy(target, drafts, ...)` finishes the round
    exactly like a greedy one. Requests with temperature <= 0 are greedy (their law is the argmax; `greedy_pick`
    int64 [B * (k + 1)], when the caller already has every row's argmax, is copied for them instead).
    Reference: hibana/kernels/sampled_verify.py:17-106, hibana/engine/rejection.py:115-186."""
    b, k = drafts.shape
    if nv.use_native(logits):
        dev = logits.device
        target = torch.empty(b, k + 1, dtype=torch.int64, device=dev)
        p_draft = torch.empty(b, k + 1, dtype=torch.float32, device=dev)
        nv.check(nv.lib().hb_spec_targets(logits.data_ptr(), logits.stride(0), b, k, logits.shape[1],
                                          int(logits.dtype == torch.float32), drafts.data_ptr(),
                                          temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                                          seeds.data_ptr(), draws.data_ptr(), nv.ptr(soft), nv.ptr(bitmask),
                                          bitmask.shape[1] if bitmask is not None else 0, nv.ptr(greedy_pick),
                                          target.data_ptr(), p_draft.data_ptr(), nv.stream()), "hb_spec_targets")
        return target, p_draft
    return spec_targets_ref(logits, drafts, temperature, top_k, top_p, seeds, draws, soft, bitmask)


def lattice_walk(cand: torch.Tensor, scores: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                 uniforms: Optional[torch.Tensor] = None):
    """Walks a block drafter's candidate lattice. cand int64 [B, k, W], scores fp32 [B, k, W (previous choice), W];
    greedy when `temperature` / `uniforms` are None or a request's temperature is <= 0, else the path is sampled
    from softmax(row / T) with uniforms fp32 [B, k]. Returns (tokens int64 [B, k], chosen candidate index int32
    [B, k], probs fp32 [B, k, W]: the law every token was drawn from on its support, estimate fp32 [B, k]: the
    unit-temperature probability of the chosen candidate). One warp per request on the GPU (W <= 32).
    Reference: hibana/kernels/draft_selection.py:14-99."""
    b, k, w = cand.shape
    if nv.use_native(scores) and w <= 32:
        dev = scores.device
        tokens = torch.empty(b, k, dtype=torch.int64, device=dev)
        chosen = torch.empty(b, k, dtype=torch.int32, device=dev)
        probs = torch.empty(b, k, w, dtype=torch.float32, device=dev)
        est = torch.empty(b, k, dtype=torch.float32, device=dev)
        scores = scores.float().contiguous()
        nv.check(nv.lib().hb_lattice_walk(cand.contiguous().data_ptr(), scores.data_ptr(), nv.ptr(temperature),
                                          nv.ptr(uniforms), b, k, w, tokens.data_ptr(), chosen.data_ptr(),
                                          probs.data_ptr(), est.data_ptr(), nv.stream()), "hb_lattice_walk")
        return tokens, chosen, probs, est
    prev = torch.zeros(b, dtype=torch.long, device=cand.device)
    toks, idxs, ps, ests = [], [], [], []
    for j in range(k):
        row = scores[:, j].float().gather(1, prev[:, None, None].expand(-1, 1, w)).squeeze(1)
        p1 = torch.softmax(row, -1)
        pick = row.argmax(-1)
        p = p1
        if temperature is not None and uniforms is not None:
            hot = temperature > 0
            pt = torch.softmax(row / temperature.clamp_min(1e-6)[:, None], -1)
            drawn = (pt.cumsum(-1) < uniforms[:, j, None]).sum(-1).clamp_max(w - 1)
            pick = torch.where(hot, drawn, pick)
            p = torch.where(hot[:, None], pt, p1)
        prev = pick
        idxs.append(pick.int())
        toks.append(cand[:, j].gather(1, pick[:, None]).squeeze(1))
        ps.append(p)
        ests.append(p1.gather(1, pick[:, None]).squeeze(1))
    return torch.stack(toks, 1), torch.stack(idxs, 1), torch.stack(ps, 1), torch.stack(ests, 1)
