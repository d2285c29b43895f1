"""Block drafter: k draft tokens from ONE forward (the "parallel drafting" proposer's model).

The block is the pending (anchor) token followed by k copies of a learned mask token. Its positions attend,
without a causal mask inside the block, to (a) a sliding window of context entries, one per committed token, whose
keys / values are projections of  embed(token) + W_f * target_hidden(token)  (so the drafter reads the target's
own features instead of recomputing them; entries are appended as tokens are committed and never rewritten), through
a learned per-head sink logit that lets a head attend to "nothing", and (b) the block itself. A 2-tap convolution
over block positions mixes each masked position with its left neighbour before the layers. The hidden state of
masked position j gives the logits of draft token j through the target's output head (shared); the W best tokens
per position are the candidates, and a low-rank bilinear form between the embeddings of consecutive candidates turns
them into a lattice: score[j, u, w] = logit[j, w] + <P e(cand[j-1, u]), Q e(cand[j, w])>, i.e. the choice at
position j is conditioned on the choice at j - 1 although all positions came from one forward. `greedy_lattice`
/ `sample_lattice` walk it. Weights are random-init here (no trained drafter checkpoint exists for this build);
speculative decoding stays exact for any drafter because every draft is verified by the target.
Reference: hibana/model/parallel_draft.py (masked positions, feature projection, 2-tap conv, sink attention,
bilinear selector), hibana/kernels/draft_selection.py (lattice walks), hibana/proposers/parallel.py:232-277.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def _rope(x: torch.Tensor, pos: torch.Tensor, theta: float = 10000.0) -> torch.Tensor:
    """x [..., T, heads, d], pos [..., T] -> rotary embedding over the last dim (pairs (i, i + d/2))."""
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d // 2, device=x.device, dtype=torch.float32) / (d // 2))
    ang = pos.float()[..., None, None] * inv                       # [..., T, 1, d/2]
    c, s = ang.cos(), ang.sin()
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


class BlockDrafter:
    def __init__(self, hidden: int, vocab: int, embed: torch.Tensor, lm_head: torch.Tensor, *, layers: int = 2,
                 heads: int = 8, width: int = 4, rank: int = 32, window: int = 256, max_depth: int = 15,
                 device="cpu", seed: int = 0, dtype=torch.float32):
        assert hidden % heads == 0 and (hidden // heads) % 2 == 0
        g = torch.Generator().manual_seed(seed)
        self.h, self.vocab, self.nl, self.nh, self.hd = hidden, vocab, layers, heads, hidden // heads
        self.width, self.window, self.max_depth = width, window, max_depth
        self.embed, self.lm_head = embed, lm_head                  # shared with the target ([V, H] each)
        self.device, self.dtype = torch.device(device), dtype

        def w(*shape, scale=None):
            scale = scale if scale is not None else 1.0 / math.sqrt(shape[-1])
            return (torch.randn(*shape, generator=g) * scale).to(self.device, dtype)

        self.mask_embed = w(hidden, scale=0.02)
        self.feat_proj = w(hidden, hidden)                         # target feature -> drafter space
        self.conv = torch.tensor([1.0, 0.25], device=self.device, dtype=dtype)   # taps: self, left neighbour
        self.layers = []
        for _ in range(layers):
            self.layers.append({
                "ln1": torch.ones(hidden, device=self.device, dtype=dtype),
                "ln2": torch.ones(hidden, device=self.device, dtype=dtype),
                "q": w(hidden, hidden), "k": w(hidden, hidden), "v": w(hidden, hidden), "o": w(hidden, hidden),
                "ck": w(hidden, hidden), "cv": w(hidden, hidden),   # context (feature) keys / values
                "sink": torch.zeros(heads, device=self.device, dtype=torch.float32),
                "up": w(4 * hidden, hidden), "down": w(hidden, 4 * hidden)})
        self.norm = torch.ones(hidden, device=self.device, dtype=dtype)
        self.sel_p, self.sel_q = w(rank, hidden), w(rank, hidden)

    # ---- context entries
    def context_kv(self, tokens: torch.Tensor, features: torch.Tensor, positions: torch.Tensor):
        """tokens [n], target hiddens [n, H], positions [n] -> per layer (K, V) [n, heads, d] of the context."""
        x = self.embed[tokens].to(self.dtype) + features.to(self.dtype) @ self.feat_proj.t()
        x = F.rms_norm(x, (self.h,))
        out = []
        for ly in self.layers:
            k = (x @ ly["ck"].t()).view(-1, self.nh, self.hd)
            v = (x @ ly["cv"].t()).view(-1, self.nh, self.hd)
            out.append((_rope(k, positions), v))
        return out

    # ---- the block forward
    def forward(self, anchors: torch.Tensor, positions: torch.Tensor, ctx_k, ctx_v, ctx_mask: torch.Tensor,
                depth: int) -> torch.Tensor:
        """anchors [B] tokens at positions [B]; ctx_k / ctx_v: per layer [B, Wn, heads, d]; ctx_mask [B, Wn] bool
        (valid context entries). Returns the hidden states of the `depth` masked positions [B, depth, H]."""
        b, s = anchors.shape[0], depth + 1
        x = self.mask_embed.expand(b, s, self.h).clone()
        x[:, 0] = self.embed[anchors].to(self.dtype)
        x = self.conv[0] * x + self.conv[1] * F.pad(x, (0, 0, 1, 0))[:, :-1]        # 2-tap conv over the block
        pos = positions[:, None] + torch.arange(s, device=x.device)
        scale = 1.0 / math.sqrt(self.hd)
        for li, ly in enumerate(self.layers):
            hn = F.rms_norm(x, (self.h,), ly["ln1"])
            q = _rope((hn @ ly["q"].t()).view(b, s, self.nh, self.hd), pos)
            k = _rope((hn @ ly["k"].t()).view(b, s, self.nh, self.hd), pos)
            v = (hn @ ly["v"].t()).view(b, s, self.nh, self.hd)
            keys = torch.cat([ctx_k[li].to(self.dtype), k], 1)                  # [B, Wn + s, heads, d]
            vals = torch.cat([ctx_v[li].to(self.dtype), v], 1)
            att = torch.einsum("bqhd,bkhd->bhqk", q.float(), keys.float()) * scale
            valid = torch.cat([ctx_mask, torch.ones(b, s, dtype=torch.bool, device=x.device)], 1)
            att = att.masked_fill(~valid[:, None, None, :], float("-inf"))
            sink = ly["sink"].view(1, self.nh, 1, 1).expand(b, -1, s, -1)       # attend-to-nothing logit
            p = torch.softmax(torch.cat([att, sink], -1), -1)[..., :-1]
            o = torch.einsum("bhqk,bkhd->bqhd", p, vals.float()).reshape(b, s, self.h).to(self.dtype)
            x = x + o @ ly["o"].t()
            hn = F.rms_norm(x, (self.h,), ly["ln2"])
            x = x + F.silu(hn @ ly["up"].t()) @ ly["down"].t()
        return F.rms_norm(x, (self.h,), self.norm)[:, 1:]

    # ---- candidates and lattice
    def select(self, hidden: torch.Tensor, anchors: torch.Tensor):
        """hidden [B, k, H] -> candidates int64 [B, k, W], scores fp32 [B, k, W (previous choice), W]."""
        logits = hidden.float() @ self.lm_head.float().t()                       # [B, k, V]
        top, cand = logits.topk(self.width, -1)
        e = self.embed[cand].float()                                            # [B, k, W, H]
        prev = torch.cat([self.embed[anchors].float()[:, None, None, :].expand(-1, 1, self.width, -1), e[:, :-1]], 1)
        pair = torch.einsum("bkur,bkwr->bkuw", prev @ self.sel_p.float().t(), e @ self.sel_q.float().t())
        return cand, top[:, :, None, :] + pair


def greedy_lattice(cand: torch.Tensor, scores: torch.Tensor):
    """Walks the lattice taking the best next candidate given the previous choice. Returns (tokens [B, k],
    chosen index [B, k])."""
    b, k, w = cand.shape
    prev = torch.zeros(b, dtype=torch.long, device=cand.device)
    toks, idxs = [], []
    for j in range(k):
        row = scores[:, j].gather(1, prev[:, None, None].expand(-1, 1, w)).squeeze(1)      # [B, W]
        prev = row.argmax(-1)
        idxs.append(prev)
        toks.append(cand[:, j].gather(1, prev[:, None]).squeeze(1))
    return torch.stack(toks, 1), torch.stack(idxs, 1)


def sample_lattice(cand: torch.Tensor, scores: torch.Tensor, temperature: torch.Tensor, uniforms: torch.Tensor,
                   vocab: int):
    """Samples a path: at each step from softmax(scores[j, previous choice, :] / T) with the given uniforms
    [B, k]. Returns (tokens [B, k], laws fp32 [B, k, vocab]: the distribution each token was drawn from, dense
    over the vocabulary as speculative sampling needs it)."""
    b, k, w = cand.shape
    prev = torch.zeros(b, dtype=torch.long, device=cand.device)
    toks = []
    laws = torch.zeros(b, k, vocab, device=cand.device)
    for j in range(k):
        row = scores[:, j].gather(1, prev[:, None, None].expand(-1, 1, w)).squeeze(1)
        p = torch.softmax(row / temperature.clamp_min(1e-6)[:, None], -1)
        laws[:, j].scatter_add_(1, cand[:, j], p)
        prev = (p.cumsum(-1) < uniforms[:, j, None]).sum(-1).clamp_max(w - 1)
        toks.append(cand[:, j].gather(1, prev[:, None]).squeeze(1))
    return torch.stack(toks, 1), laws
