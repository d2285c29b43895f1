"""LiLiCorr drafter: the block drafter with dynamic two-tap convolutions and a learned candidate-lattice scorer.

Where the plain block drafter (models/parallel_draft.py) scores the lattice with one bilinear form between the
embeddings of consecutive candidates, LiLiCorr runs a small transformer ("correlator") over all slots x top-k
candidates of a block at once and reads transition scores from it:

    per candidate   x = W_tok e(token) + W_hid h(slot) + MLP(LayerNorm([log p, p, log p - max, rank, is_top]))
                        + slot embedding + rank embedding
    layers          pre-norm attention over the slots * topk candidates with a learned bias per head that depends
                    on the slot distance (plus a same-slot term), then a SiLU MLP
    factors         f = SiLU(W [x, a, x * a]) with a = norm(W_ctx anchor feature) the request's context vector
    heads           out(f), in(f), unit-normalised; score[j, u, w] = scale * <out[j - 1, u], in[j, w]>,
                    score[0, :, w] = scale * <anchor_out(a), in[0, w]>

and the grouped two-tap convolution mixes each block position with its left neighbour in groups of 16 features,
with coefficients base + W_kernel h (two taps, applied before and after the layers). The lattice is then walked
exactly like the block drafter's (ops/sampling.py `lattice_walk`), so the proposer, the verify round and the
acceptance rules are shared. Weights are random-init (no trained checkpoint exists offline); every draft is verified
by the target, so decoding stays exact whatever the drafter proposes.
Reference: hibana/model/lilicorr.py:21-163 (convolve, correlate, selector), hibana/model/lilicorr_config.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .parallel_draft import BlockDrafter


def two_tap_conv(x: torch.Tensor, coeff: torch.Tensor, base: torch.Tensor) -> torch.Tensor:
    """x [B, S, H]; coeff [B, S, 2, H / 16] (per position and 16-feature group); base [2, H]. Output position s is
    (base0 + c0) * x[s] + (base1 + c1) * x[s - 1] with fp32 coefficients (position 0 has no left neighbour)."""
    b, s, h = x.shape
    g = x.float().view(b, s, h // 16, 16)
    prev = F.pad(g[:, :-1], (0, 0, 0, 0, 1, 0))
    c = base.float().view(1, 1, 2, h // 16, 16) + coeff.float().unsqueeze(-1)
    return (c[:, :, 0] * g + c[:, :, 1] * prev).flatten(-2).to(x.dtype)


class LiLiCorrDrafter(BlockDrafter):
    def __init__(self, hidden: int, vocab: int, embed: torch.Tensor, lm_head: torch.Tensor, *, topk: int = 4,
                 corr_hidden: int = 128, corr_heads: int = 4, corr_layers: int = 2, factor_dim: int = 64,
                 logit_scale: float = 4.0, block_size: int = 16, **kw):
        assert hidden % 16 == 0 and corr_hidden % corr_heads == 0
        super().__init__(hidden, vocab, embed, lm_head, width=topk, **kw)
        g = torch.Generator().manual_seed(kw.get("seed", 0) + 101)
        self.ch, self.cheads, self.block_size, self.logit_scale = corr_hidden, corr_heads, block_size, logit_scale

        def w(*shape, scale=None):
            scale = scale if scale is not None else 1.0 / math.sqrt(shape[-1])
            return (torch.randn(*shape, generator=g) * scale).to(self.device, self.dtype)

        h, c = hidden, corr_hidden
        self.kernel_proj = w(2 * 2 * (h // 16), h, scale=0.01)            # [pre | post] x [tap] x groups
        self.base_kernel = torch.zeros(2, 2, h, device=self.device, dtype=self.dtype)
        self.base_kernel[:, 0] = 1.0                                       # identity tap, small learned deviations
        self.base_kernel[:, 1] = 0.25
        self.corr = {
            "feat_norm_w": torch.ones(5, device=self.device, dtype=self.dtype),
            "feat_norm_b": torch.zeros(5, device=self.device, dtype=self.dtype),
            "feat_up": w(c, 5), "feat_down": w(c, c), "tok": w(c, h), "hid": w(c, h), "ctx": w(c, h),
            "slot_emb": w(block_size, c, scale=0.02), "rank_emb": w(topk, c, scale=0.02),
            "rel_bias": w(corr_heads, 2 * block_size - 1, scale=0.1), "same_bias": w(corr_heads, scale=0.1),
            "out_norm": torch.ones(c, device=self.device, dtype=self.dtype),
            "anchor_norm": torch.ones(c, device=self.device, dtype=self.dtype),
            "factor_in": w(factor_dim, 3 * c), "out_head": w(factor_dim, factor_dim), "in_head": w(factor_dim, factor_dim),
            "anchor_out": w(factor_dim, c),
            "layers": [{"n1": torch.ones(c, device=self.device, dtype=self.dtype),
                        "n2": torch.ones(c, device=self.device, dtype=self.dtype),
                        "qkv": w(3 * c, c), "qkv_b": torch.zeros(3 * c, device=self.device, dtype=self.dtype),
                        "o": w(c, c), "up": w(2 * c, c), "down": w(c, 2 * c)} for _ in range(corr_layers)],
        }
        self._anchor_feat = None

    # ---- block forward with the dynamic convolutions around the layers
    def forward(self, anchors, positions, ctx_k, ctx_v, ctx_mask, depth):
        b, s = anchors.shape[0], depth + 1
        x = self.mask_embed.expand(b, s, self.h).clone()
        x[:, 0] = self.embed[anchors].to(self.dtype)
        coeff = (x @ self.kernel_proj.t()).view(b, s, 2, 2, self.h // 16)
        x = two_tap_conv(x, coeff[:, :, 0], self.base_kernel[0])
        pos = positions[:, None] + torch.arange(s, device=x.device)
        scale = 1.0 / math.sqrt(self.hd)
        from .parallel_draft import _rope
        for li, ly in enumerate(self.layers):
            hn = F.rms_norm(x, (self.h,), ly["ln1"])
            q = _rope((hn @ ly["q"].t()).view(b, s, self.nh, self.hd), pos)
            k = _rope((hn @ ly["k"].t()).view(b, s, self.nh, self.hd), pos)
            v = (hn @ ly["v"].t()).view(b, s, self.nh, self.hd)
            keys = torch.cat([ctx_k[li].to(self.dtype), k], 1)
            vals = torch.cat([ctx_v[li].to(self.dtype), v], 1)
            att = torch.einsum("bqhd,bkhd->bhqk", q.float(), keys.float()) * scale
            valid = torch.cat([ctx_mask, torch.ones(b, s, dtype=torch.bool, device=x.device)], 1)
            att = att.masked_fill(~valid[:, None, None, :], float("-inf"))
            sink = ly["sink"].view(1, self.nh, 1, 1).expand(b, -1, s, -1)
            p = torch.softmax(torch.cat([att, sink], -1), -1)[..., :-1]
            o = torch.einsum("bhqk,bkhd->bqhd", p, vals.float()).reshape(b, s, self.h).to(self.dtype)
            x = x + o @ ly["o"].t()
            hn = F.rms_norm(x, (self.h,), ly["ln2"])
            x = x + F.silu(hn @ ly["up"].t()) @ ly["down"].t()
        x = two_tap_conv(x, coeff[:, :, 1], self.base_kernel[1])
        out = F.rms_norm(x, (self.h,), self.norm)
        self._anchor_feat = out[:, 0]                    # the anchor position's state: the request's context vector
        return out[:, 1:]

    # ---- the correlator
    def correlate(self, emb: torch.Tensor, logp: torch.Tensor, hidden: torch.Tensor, anchor: torch.Tensor):
        """emb [B, k, W, H] candidate embeddings, logp [B, k, W] their log-probabilities (descending), hidden
        [B, k, H], anchor [B, H]. Returns transition scores fp32 [B, k, W (previous choice), W]."""
        c = self.corr
        b, k, wd = logp.shape
        if k > self.block_size:
            raise ValueError(f"draft length {k} exceeds the {self.block_size} slots the correlator knows")
        rank = torch.arange(wd, device=logp.device, dtype=torch.float32) / max(wd - 1, 1)
        feats = torch.stack([logp, logp.exp(), logp - logp.amax(-1, keepdim=True), rank.expand_as(logp),
                             (rank == 0).float().expand_as(logp)], -1).to(self.dtype)
        feats = F.layer_norm(feats, (5,), c["feat_norm_w"], c["feat_norm_b"])
        x = emb.to(self.dtype) @ c["tok"].t() + (hidden.to(self.dtype) @ c["hid"].t()).unsqueeze(-2)
        x = x + F.silu(feats @ c["feat_up"].t()) @ c["feat_down"].t()
        x = x + c["slot_emb"][:k, None, :] + c["rank_emb"][None, :wd, :]
        x = x.flatten(1, 2)                                                 # [B, k * W, C]
        slots = torch.arange(k, device=x.device).repeat_interleave(wd)
        rel = slots[:, None] - slots[None, :]
        bias = c["rel_bias"][:, rel + self.block_size - 1] + (rel == 0) * c["same_bias"][:, None, None]
        hd = self.ch // self.cheads
        for ly in c["layers"]:
            n = F.rms_norm(x, (self.ch,), ly["n1"])
            qkv = F.linear(n, ly["qkv"], ly["qkv_b"]).view(b, k * wd, 3, self.cheads, hd)
            q, kk, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            att = F.scaled_dot_product_attention(q.float(), kk.float(), v.float(), attn_mask=bias[None].float())
            x = x + att.transpose(1, 2).reshape(b, k * wd, self.ch).to(self.dtype) @ ly["o"].t()
            n = F.rms_norm(x, (self.ch,), ly["n2"])
            x = x + F.silu(n @ ly["up"].t()) @ ly["down"].t()
        x = F.rms_norm(x, (self.ch,), c["out_norm"]).view(b, k, wd, self.ch)
        a = F.rms_norm(anchor.to(self.dtype) @ c["ctx"].t(), (self.ch,), c["anchor_norm"])
        row = a[:, None, None].expand_as(x)
        f = F.silu(torch.cat([x, row, x * row], -1) @ c["factor_in"].t())
        out_v = F.normalize((f @ c["out_head"].t()).float(), dim=-1, eps=1e-6)
        in_v = F.normalize((f @ c["in_head"].t()).float(), dim=-1, eps=1e-6)
        a_out = F.normalize((a @ c["anchor_out"].t()).float(), dim=-1, eps=1e-6)
        start = (a_out[:, None] * in_v[:, 0]).sum(-1)                       # [B, W]
        pairs = out_v[:, :-1] @ in_v[:, 1:].transpose(-1, -2)               # [B, k - 1, W, W]
        return torch.cat([start[:, None, None].expand(-1, 1, wd, -1), pairs], 1) * self.logit_scale

    def select(self, hidden: torch.Tensor, anchors: torch.Tensor):
        """hidden [B, k, H] -> (candidates int64 [B, k, W], scores fp32 [B, k, W, W]): a slot's candidates are its W
        most likely tokens; the score of candidate w after previous choice u is its log-probability plus the
        correlator's transition term."""
        logits = hidden.float() @ self.lm_head.float().t()
        logp, cand = logits.log_softmax(-1).topk(self.width, -1)
        anchor = self._anchor_feat if self._anchor_feat is not None else hidden[:, 0]
        trans = self.correlate(self.embed[cand], logp, hidden, anchor)
        return cand, logp[:, :, None, :] + trans
