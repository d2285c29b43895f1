"""Speculative sampling (sampled acceptance) for non-greedy requests.

For a verified block [pending, d_1 .. d_k] with target distributions p_0 .. p_k (p_j = law of the token after row j)
and draft laws q_1 .. q_k:
  * draft d_{j+1} is accepted with probability min(1, p_j[d] / q_{j+1}[d]); with slack s > 0 (`accept_soft`) it is
    also accepted when u * q[d] < e^s * p[d] on the SAME uniform draw u;
  * at the first rejection the replacement is drawn from the residual max(p_j - q_{j+1}, 0) renormalised, and no
    target draw past that row is consumed;
  * after k acceptances the bonus token is drawn from p_k.
The emitted sequence is then distributed exactly as sampling from the target alone (s = 0). Both laws are the
distributions actually sampled from: temperature, top-k and top-p (nucleus) are applied first (`distribution`).
Every random number comes from the request's counter-based generator: `uniforms[j]` decides row j and
`residual_uniforms[j]` inverts the residual / bonus CDF, so a replayed round makes the same choices.
`verify_batch` is the vectorised form (torch ops only, runs on the logits' device without host loops);
`verify_row` is the per-row statement of the rule and the tests' oracle.
Reference: hibana/engine/rejection.py:68-367, docs/interfaces.md:163-172.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch


def distribution(logits: torch.Tensor, temperature: float | torch.Tensor, top_k: int | torch.Tensor = 0,
                 top_p: float | torch.Tensor = 1.0) -> torch.Tensor:
    """Rows of probabilities after temperature, top-k and nucleus truncation (per-row parameters allowed).
    temperature <= 0 gives the one-hot argmax law."""
    lg = logits.float()
    rows, vocab = lg.shape
    dev = lg.device
    temp = torch.as_tensor(temperature, dtype=torch.float32, device=dev).expand(rows).clone()
    k = torch.as_tensor(top_k, dtype=torch.int64, device=dev).expand(rows).clone()
    p = torch.as_tensor(top_p, dtype=torch.float32, device=dev).expand(rows)
    greedy = temp <= 0
    temp[greedy] = 1.0
    k[(k <= 0) | (k > vocab)] = vocab
    k[greedy] = 1
    srt, idx = torch.sort(lg / temp[:, None], dim=-1, descending=True, stable=True)
    ranks = torch.arange(vocab, device=dev)[None, :]
    srt = srt.masked_fill(ranks >= k[:, None], float("-inf"))
    probs = torch.softmax(srt, dim=-1)
    # nucleus: keep the smallest prefix whose mass reaches top_p (the token that crosses the line stays)
    csum = probs.cumsum(-1)
    keep = (csum - probs) < p[:, None]
    keep[:, 0] = True
    probs = torch.where(keep, probs, torch.zeros_like(probs))
    probs = probs / probs.sum(-1, keepdim=True)
    out = torch.zeros_like(probs)
    out.scatter_(1, idx, probs)
    return out


def _inverse_cdf(law: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Smallest index whose cumulative mass exceeds u (rows of `law` sum to 1)."""
    c = law.cumsum(-1)
    c[:, -1] = 1.0 + 1e-6
    return (c <= u[:, None]).sum(-1).clamp_max(law.shape[1] - 1)


def verify_row(p: Sequence[torch.Tensor], q: Sequence[torch.Tensor], drafts: Sequence[int], uniforms: Sequence[float],
               residual_uniforms: Sequence[float], soft: float = 0.0) -> tuple[list[int], int]:
    """One request. p: k + 1 target laws, q: k draft laws. Returns (emitted tokens, accepted drafts)."""
    out = []
    for j, d in enumerate(drafts):
        pj, qj = float(p[j][d]), float(q[j][d])
        u = uniforms[j]
        ok = qj > 0 and (u * qj < pj or (soft > 0 and u * qj < math.exp(soft) * pj))
        if not ok:
            res = (p[j] - q[j]).clamp_min(0)
            res = res / res.sum() if float(res.sum()) > 0 else p[j]
            out.append(int(_inverse_cdf(res[None, :], torch.tensor([residual_uniforms[j]]))[0]))
            return out, j
        out.append(int(d))
    k = len(drafts)
    out.append(int(_inverse_cdf(p[k][None, :], torch.tensor([residual_uniforms[k]]))[0]))
    return out, k


@dataclass
class Verdict:
    emitted: torch.Tensor     # int64 [B, k + 1], valid up to count
    count: torch.Tensor       # int32 [B] tokens emitted (accepted + 1)
    accepted: torch.Tensor    # int32 [B]


def verify_batch(target_laws: torch.Tensor, draft_laws: torch.Tensor, drafts: torch.Tensor, uniforms: torch.Tensor,
                 residual_uniforms: torch.Tensor, soft: float | torch.Tensor = 0.0) -> Verdict:
    """target_laws [B, k + 1, V], draft_laws [B, k, V], drafts int64 [B, k], uniforms / residual_uniforms fp32
    [B, k + 1]. Vectorised over the batch and the block; nothing leaves the device."""
    b, k1, v = target_laws.shape
    k = k1 - 1
    dev = target_laws.device
    soft_t = torch.as_tensor(soft, dtype=torch.float32, device=dev).expand(b)
    pd = target_laws[:, :k].gather(2, drafts[:, :, None]).squeeze(2)
    qd = draft_laws.gather(2, drafts[:, :, None]).squeeze(2)
    u = uniforms[:, :k]
    ok = (qd > 0) & ((u * qd < pd) | ((soft_t[:, None] > 0) & (u * qd < torch.exp(soft_t)[:, None] * pd)))
    accepted = torch.cumprod(ok.to(torch.int32), dim=1).sum(1)                  # longest accepted prefix
    row = accepted.clamp_max(k)                                                  # row that draws the last token
    p_row = target_laws[torch.arange(b, device=dev), row]
    q_row = draft_laws[torch.arange(b, device=dev), row.clamp_max(max(k - 1, 0))] if k else torch.zeros_like(p_row)
    res = (p_row - q_row).clamp_min(0)
    rs = res.sum(-1, keepdim=True)
    res = torch.where(rs > 0, res / rs.clamp_min(1e-30), p_row)
    law = torch.where((accepted == k)[:, None], p_row, res)                     # bonus draw after full acceptance
    last = _inverse_cdf(law, residual_uniforms[torch.arange(b, device=dev), row])
    emitted = torch.cat([drafts, torch.zeros(b, 1, dtype=drafts.dtype, device=dev)], 1)
    emitted[torch.arange(b, device=dev), row] = last
    return Verdict(emitted, (accepted + 1).to(torch.int32), accepted.to(torch.int32))


def relaxed_greedy(rank: torch.Tensor, gap: torch.Tensor, top_k: int, margin: float) -> torch.Tensor:
    """Relaxed greedy acceptance: the drafted token counts as matching when it is within the target's top-K and
    within `margin` logits of the argmax (rank 0 = the argmax itself). rank int32 / gap fp32 [B, k]."""
    return (rank < max(top_k, 1)) & ((gap <= margin) | (rank == 0))
