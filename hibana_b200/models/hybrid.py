"""Hybrid decoder families built from the layer library: tiny hybrid MoE, the reference's 27B (gated delta rule +
gated attention), Flash-Next-class (plus MoE) and Nemotron-class (Mamba-2 / latent MoE / attention blocks by
pattern). A block is (mixer, ffn) with either part optional; every sublayer is pre-norm with a residual stream.

Reference: hibana/model/qwen38.py:53-184, hibana/model/flashnext/model.py:42-277,
hibana/model/nemotron/model.py:71-280.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..engine.context import ForwardContext
from ..ops import basic, gemm
from ..target import GDN, MAMBA2, NONE, Target
from .layers import Init, MoeLayer, build_ffn, build_mixer


class Block:
    def __init__(self, t: Target, init: Init, idx: int, mixer_kind: str, ffn_kind: str, counters: dict,
                 ep_rank: int, ep_size: int):
        self.mixer = build_mixer(mixer_kind, t, init, counters, f"l{idx}.mixer")
        self.ffn = build_ffn(ffn_kind, t, init, f"l{idx}.ffn", ep_rank, ep_size)
        self.mixer_norm = init.ones(t.hidden, t.gemma_norm) if self.mixer is not None else None
        self.ffn_norm = init.ones(t.hidden, t.gemma_norm) if self.ffn is not None else None

    def sublayers(self):
        return [(self.mixer_norm, self.mixer), (self.ffn_norm, self.ffn)]


class HybridModel:
    def __init__(self, t: Target, device="cpu", seed: int = 0, init_device=None, ep_rank: int = 0, ep_size: int = 1):
        self.target = t
        self.device = torch.device(device)
        init = Init(seed, self.device, init_device)
        self.embed = init.normal(t.vocab, t.hidden).to(torch.bfloat16).to(self.device)
        counters = {"kv": 0, "state": 0}
        self.blocks = [Block(t, init, i, m, f, counters, ep_rank, ep_size) for i, (m, f) in enumerate(t.layers)]
        self.final_norm = init.ones(t.hidden, t.gemma_norm)
        self.lm_head = self.embed if t.tie_embeddings else init.normal(t.vocab, t.hidden).to(torch.bfloat16).to(
            self.device)
        self.kv_layers, self.state_layers = counters["kv"], counters["state"]
        self.ep_size = ep_size
        # Hyper-connections: one site in front of every sublayer (its gated mix of the residual streams is the
        # sublayer's input, the sublayer's output is injected back into every stream) and a last site, without
        # injection, in front of the final norm.
        self.hyper_sites = None
        if t.hyper_streams > 1:
            from .hyper import HyperConnection
            hc, hh, rk = t.hyper_streams, t.hidden, t.hyper_rank
            n_sites = sum(1 for b in self.blocks for _, sub in b.sublayers() if sub is not None) + 1
            self.hyper_sites = []
            for i in range(n_sites):
                last = i == n_sites - 1
                self.hyper_sites.append(HyperConnection(
                    init.ones(hc * hh, True).to(self.device), init.normal(rk, hc * hh).to(self.device),
                    init.normal(hc * hh, rk).to(self.device),
                    None if last else init.normal(hc, hc * hh).to(self.device), hc, hh, t.norm_eps))
        self.mtp = None
        if t.mtp_layers:
            from .mtp import MtpHead
            self.mtp = MtpHead(t, init, self)

    # ---- bookkeeping
    def linears(self):
        out = []
        for b in self.blocks:
            for _, sub in b.sublayers():
                if sub is not None:
                    out += sub.linears()
        return out

    def state_pool_spec(self) -> Optional[dict]:
        """Shape of the recurrent-state pool this model needs (None = attention only)."""
        t = self.target
        kinds = {m for m, _ in t.layers}
        if MAMBA2 in kinds:
            return {"layers": self.state_layers, "conv_dim": t.mamba_conv_dim, "conv_width": t.conv_width,
                    "state_shape": (t.mamba_heads, t.mamba_head_dim, t.mamba_state)}
        if GDN in kinds:
            return {"layers": self.state_layers, "conv_dim": t.gdn_conv_dim, "conv_width": t.conv_width,
                    "state_shape": (t.gdn_v_heads, t.gdn_head_dim, t.gdn_head_dim)}
        return None

    def calibrate(self, run_forward, comm=None) -> None:
        lins = [lin for lin in self.linears() if lin.fmt == "nvfp4"]
        for lin in lins:
            lin.calibrating, lin.seen_amax = True, 0.0
        try:
            run_forward()
        finally:
            for lin in lins:
                lin.calibrating = False
        for lin in lins:
            lin.set_input_amax(max(lin.seen_amax, 1e-3) * 1.5)

    # ---- forward
    def hidden_states(self, ids: torch.Tensor, ctx: ForwardContext, kv, states=None):
        """Runs the trunk; returns (h, res) of the last sublayer (the final norm adds them)."""
        t = self.target
        if self.hyper_sites is not None:
            return self._hidden_states_hyper(ids, ctx, kv, states)
        res = basic.embedding(ids, self.embed)
        h: Optional[torch.Tensor] = None
        for blk in self.blocks:
            for norm_w, sub in blk.sublayers():
                if sub is None:
                    continue
                x = basic.rmsnorm(res if h is None else h, norm_w, t.norm_eps,
                                  residual=None if h is None else res, gemma=t.gemma_norm)
                if isinstance(sub, MoeLayer) and ctx.extras.get("ep") is not None:
                    # data-parallel attention + expert-parallel experts: this rank's own tokens travel to the
                    # owners of their experts and back (parallel/ep.py); every rank runs every layer each step
                    h = sub.forward_a2a(x, ctx.extras["ep"])
                elif isinstance(sub, MoeLayer) and sub.ep_size > 1 and ctx.comm is not None:
                    h = sub.forward_ep(x, ctx.comm)
                else:
                    h = sub.forward(x, ctx, kv, states)
        return h, res

    def _run_sublayer(self, sub, x, ctx, kv, states):
        if isinstance(sub, MoeLayer) and ctx.extras.get("ep") is not None:
            return sub.forward_a2a(x, ctx.extras["ep"])
        if isinstance(sub, MoeLayer) and sub.ep_size > 1 and ctx.comm is not None:
            return sub.forward_ep(x, ctx.comm)
        return sub.forward(x, ctx, kv, states)

    def _hidden_states_hyper(self, ids: torch.Tensor, ctx: ForwardContext, kv, states=None):
        """Trunk with hyper-connections: the token's state is `hyper_streams` residual streams [T, hc * H]; a site's
        per-stream norm and gated mean stand where the pre-norm + residual add stand in the plain trunk.
        Reference: hibana/model/flashnext/model.py:42-77."""
        t = self.target
        hyper = basic.embedding(ids, self.embed).repeat(1, t.hyper_streams)
        site = 0
        for blk in self.blocks:
            for _norm_w, sub in blk.sublayers():
                if sub is None:
                    continue
                hc = self.hyper_sites[site]
                site += 1
                x, keep = hc.mix(hyper)
                hyper = hc.combine(self._run_sublayer(sub, x, ctx, kv, states), keep)
        x, _ = self.hyper_sites[site].mix(hyper)
        return x, torch.zeros_like(x)

    def forward(self, ids: torch.Tensor, ctx: ForwardContext, kv, states=None) -> torch.Tensor:
        t = self.target
        h, res = self.hidden_states(ids, ctx, kv, states)
        if ctx.extras.get("want_hidden") is not None:
            # pre-norm hidden state of every row (feature for the MTP drafter): h + res
            ctx.extras["hidden"] = basic.add(h, res)
        if ctx.sample_rows is not None:
            h = h.index_select(0, ctx.sample_rows)
            res = res.index_select(0, ctx.sample_rows)
        return basic.rmsnorm(h, self.final_norm, t.norm_eps, residual=res, gemma=t.gemma_norm)

    def logits(self, normed: torch.Tensor, comm=None) -> torch.Tensor:
        return gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
