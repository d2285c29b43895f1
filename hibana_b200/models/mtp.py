"""Multi-token-prediction draft head: one decoder layer on top of the target's hidden states.

Input at position p is the pair (target hidden h_p, embedding of the next token x_{p+1}); the output predicts
x_{p+2}. It keeps its own KV in an extra layer of the target's KV pool (same slots, same block table) and shares
the target's embedding and lm_head. Chaining its own output hidden drafts several tokens.
Reference: hibana/model/mtp.py:1-67, hibana/model/mtp_layer.py:1-92, hibana/model/flashnext/mtp.py:1-132.
"""
from __future__ import annotations

import torch

from ..engine.context import ForwardContext
from ..ops import basic, gemm
from ..target import ATTN, MLP, Target
from .layers import AttentionLayer, Init, MlpLayer


class MtpHead:
    def __init__(self, t: Target, init: Init, base):
        self.t, self.base = t, base
        self.enorm = init.ones(t.hidden, t.gemma_norm)
        self.hnorm = init.ones(t.hidden, t.gemma_norm)
        self.fc = init.linear(t.hidden, 2 * t.hidden, "bf16", "mtp.fc")
        self.attn = AttentionLayer(t, init, base.kv_layers, False, "mtp.attn")
        f = init.full or t
        width = f.ffn or max(f.expert_ffn * max(f.top_k, 1) // 2, 128)       # unsharded width (MlpLayer splits it)
        self.mlp = MlpLayer(t, init, "mtp.mlp", width=width)
        self.attn_norm = init.ones(t.hidden, t.gemma_norm)
        self.mlp_norm = init.ones(t.hidden, t.gemma_norm)
        self.final_norm = init.ones(t.hidden, t.gemma_norm)

    def linears(self):
        return [self.fc] + self.attn.linears() + self.mlp.linears()

    def forward(self, hidden: torch.Tensor, next_ids: torch.Tensor, ctx: ForwardContext, kv):
        """hidden [T, H] (pre-norm target or previous draft hidden), next_ids int64 [T].
        Returns (chained hidden [T, H], normed [T, H] for the shared lm_head)."""
        t = self.t
        e = basic.rmsnorm(basic.embedding(next_ids, self.base.embed), self.enorm, t.norm_eps, gemma=t.gemma_norm)
        h = basic.rmsnorm(hidden, self.hnorm, t.norm_eps, gemma=t.gemma_norm)
        res = self.fc(torch.cat((e, h), dim=-1))
        x = basic.rmsnorm(res, self.attn_norm, t.norm_eps, gemma=t.gemma_norm)
        a = self.attn.forward(x, ctx, kv, None)
        tp = getattr(self.attn, "partial", False) and ctx.comm is not None
        if tp:                                   # tensor parallel: the head's two partial sums are all-reduced
            a = ctx.comm.all_reduce(a)
        x = basic.rmsnorm(a, self.mlp_norm, t.norm_eps, residual=res, gemma=t.gemma_norm)
        m = self.mlp.forward(x)
        if tp:
            m = ctx.comm.all_reduce(m)
        out = basic.add(m, res)
        return out, basic.rmsnorm(out, self.final_norm, t.norm_eps, gemma=t.gemma_norm)
