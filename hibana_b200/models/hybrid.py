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
from .. import _native as nv
from ..ops import basic, gemm, nvfp4
from ..target import GDN, MAMBA2, NONE, Target
from .layers import Init, MoeLayer, build_ffn, build_mixer


class Block:
    def __init__(self, t: Target, init: Init, idx: int, mixer_kind: str, ffn_kind: str, counters: dict,
                 ep_rank: int, ep_size: int):
        self.mixer = build_mixer(mixer_kind, t, init, counters, f"l{idx}.mixer")
        self.ffn = build_ffn(ffn_kind, t.block(idx), init, f"l{idx}.ffn", ep_rank, ep_size)
        self.mixer_norm = init.ones(t.hidden, t.gemma_norm) if self.mixer is not None else None
        self.ffn_norm = init.ones(t.hidden, t.gemma_norm) if self.ffn is not None else None

    def sublayers(self):
        return [(self.mixer_norm, self.mixer), (self.ffn_norm, self.ffn)]


class HybridModel:
    def __init__(self, t: Target, device="cpu", seed: int = 0, init_device=None, ep_rank: int = 0, ep_size: int = 1,
                 full: Optional[Target] = None):
        """`t` is this rank's geometry (`Target.shard`), `full` the unsharded target the weights are drawn from
        (same seeded stream on every rank; a rank keeps its heads / columns / experts)."""
        self.target = t
        self.full = full = full or t
        self.device = torch.device(device)
        init = Init(seed, self.device, init_device, tp=t.tp_size, rank=t.tp_rank, full=full)
        self.embed = init.normal(t.vocab, t.hidden).to(torch.bfloat16).to(self.device)
        counters = {"kv": 0, "state": 0}
        self.blocks = [Block(t, init, i, m, f, counters, ep_rank, ep_size) for i, (m, f) in enumerate(t.layers)]
        self.final_norm = init.ones(t.hidden, t.gemma_norm)
        head = self.embed if t.tie_embeddings else init.normal(t.vocab, t.hidden).to(torch.bfloat16).to(self.device)
        # vocab-parallel head under tensor parallelism: each rank scores vocab / tp tokens
        tp, rank = t.tp_size, t.tp_rank
        self.vocab_shard = t.vocab // tp if tp > 1 and t.vocab % tp == 0 else 0
        self.lm_head = head[rank * self.vocab_shard:(rank + 1) * self.vocab_shard].contiguous() \
            if self.vocab_shard else head
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
        # per-layer n-gram embedding (models/ple.py): added to the streams in front of the listed blocks
        self.ple = {}
        # (it reads and writes the hyper-connection streams: a copy of the target without streams runs without it)
        if t.ple_layers and self.hyper_sites is not None:
            from .ple import PleLayer
            self.ple = {i: PleLayer(t, init, f"blocks.{i}.ple") for i in t.ple_layers if i < len(self.blocks)}
        self.mtp = None
        if t.mtp_layers:
            from .mtp import MtpHead
            self.mtp = MtpHead(t, init, self)
        # vision encoder (targets that take images): built on first use, replicated on every rank
        self.vision_cfg = None
        self._vision = None
        self._seed = seed
        if t.vision:
            from .vision import VisionConfig
            image, patch, width, depth, heads, mlp = t.vision
            self.vision_cfg = VisionConfig(image=image, patch=patch, width=width, depth=depth, heads=heads, mlp=mlp,
                                           out_hidden=t.hidden)

    @property
    def vision(self):
        """The vision encoder, or None for a text-only target (reference: hibana/model/nemotron/vision.py:91)."""
        if self.vision_cfg is not None and self._vision is None:
            from .vision import VisionEncoder
            self._vision = VisionEncoder(self.vision_cfg, self.device, seed=self._seed + 7)
        return self._vision

    def embed_tokens(self, ids: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        """Token embeddings; rows at negative ids (image placeholders) take the vision encoder's rows handed over
        in ctx.extras["image_embeds"], in order."""
        img = ctx.extras.get("image_embeds") if ctx.extras else None
        if img is None:
            return basic.embedding(ids, self.embed)
        from ..engine.media import splice_embeddings
        return splice_embeddings(ids, basic.embedding(ids.clamp_min(0), self.embed), img.to(self.device))

    @classmethod
    def sharded(cls, full: Target, tp: int, rank: int, device, seed: int = 0, init_device=None) -> "HybridModel":
        """Tensor-parallel shard: mixers split by head, dense / shared MLPs by column, routed experts by expert
        range over the same ranks (activations are replicated, so the experts need no all-to-all), vocabulary
        split for the head. Reference: hibana/weights/sharding.py:31-88, hibana/model/flashnext/model.py:70-73."""
        ep = tp if full.experts and full.experts % tp == 0 else 1
        return cls(full.shard(tp, rank), device, seed, init_device, ep_rank=rank if ep > 1 else 0, ep_size=ep,
                   full=full)

    # ---- bookkeeping
    def linears(self):
        out = []
        for b in self.blocks:
            for _, sub in b.sublayers():
                if sub is not None:
                    out += sub.linears()
        return out

    def attach_w3(self) -> int:
        """3-bit decode copies (settings `w3`) of every NVFP4 / bf16 projection whose shape the 3-bit kernel tiles and
        of every MoE layer's routed experts: decode- and verify-sized calls stream 4 bits per weight, prefill keeps
        the served formats. Returns the bytes the copies add. Reference: hibana/kernels/w3.py `attach_model`."""
        from .linear import Linear
        added = 0
        for lin in self.linears():
            if type(lin) is not Linear or lin.in_features % 64 or lin.fmt not in ("bf16", "nvfp4"):
                continue
            if lin.name.endswith(".router"):
                continue            # fp32 logits: routing decisions stay those of the served weights
            lin.attach_w3()
            added += lin.w3.nbytes()
        for blk in self.blocks:
            if isinstance(blk.ffn, MoeLayer):
                added += blk.ffn.attach_w3()
        return added

    def state_pool_spec(self) -> Optional[dict]:
        """Shape of the recurrent-state pool this model needs (None = attention only)."""
        t = self.target
        kinds = {m for m, _ in t.layers}
        if MAMBA2 in kinds:
            return {"layers": self.state_layers, "conv_dim": t.mamba_conv_dim, "conv_width": t.conv_width,
                    "state_shape": (t.mamba_heads, t.mamba_head_dim, t.mamba_state), "groups": t.mamba_groups}
        if GDN in kinds:
            return {"layers": self.state_layers, "conv_dim": t.gdn_conv_dim, "conv_width": t.conv_width,
                    "state_shape": (t.gdn_v_heads, t.gdn_head_dim, t.gdn_head_dim), "groups": t.gdn_k_heads}
        return None

    def register_state(self, pool) -> None:
        """Per-slot state beyond the recurrences' own (called once, before any graph is captured)."""
        for layer in self.ple.values():
            layer.register(pool)

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
        res = self.embed_tokens(ids, ctx)
        h: Optional[torch.Tensor] = None
        partial = False          # h is this rank's partial sum (tensor parallel): reduced with the next norm
        for blk in self.blocks:
            for norm_w, sub in blk.sublayers():
                if sub is None:
                    continue
                xq = None
                first = getattr(sub, "first", None)
                if partial:
                    x = self._reduce_norm(h, res, norm_w, ctx)
                elif (first is not None and first.fmt == "nvfp4" and not first.calibrating and t.hidden <= 8192
                      and nv.use_native(res) and not first.takes_w3(res.shape[0])):
                    # the norm writes the first projection's NVFP4 input itself (one kernel instead of norm + quantise)
                    xq, x = nvfp4.rmsnorm_quantize(res if h is None else h, norm_w, t.norm_eps, first.input_scale,
                                                   residual=None if h is None else res, gemma=t.gemma_norm,
                                                   want_normed=sub.needs_x)
                else:
                    x = basic.rmsnorm(res if h is None else h, norm_w, t.norm_eps,
                                      residual=None if h is None else res, gemma=t.gemma_norm)
                partial = bool(getattr(sub, "partial", False)) and ctx.comm is not None
                if isinstance(sub, MoeLayer) and ctx.extras.get("ep") is not None:
                    # data-parallel attention + expert-parallel experts: this rank's own tokens travel to the
                    # owners of their experts and back (parallel/ep.py); every rank runs every layer each step
                    h = sub.forward_a2a(x, ctx.extras["ep"])
                elif isinstance(sub, MoeLayer) and sub.ep_size > 1 and ctx.comm is not None:
                    h = sub.forward_ep(x, ctx.comm)
                elif xq is not None:
                    h = sub.forward(x, ctx, kv, states, xq=xq)
                else:
                    h = sub.forward(x, ctx, kv, states)
        if partial:
            h = ctx.comm.all_reduce(h)
        return h, res

    def _reduce_norm(self, h, res, norm_w, ctx):
        """rmsnorm(all_reduce(h) + res) with `res` updated in place: one fused peer-memory kernel when the
        communicator has one and the message fits its slot, else NCCL all-reduce + the local norm."""
        t = self.target
        comm = ctx.comm
        rows = h.shape[0]
        if getattr(comm, "fused", False) and comm.fits(rows, t.hidden):
            slot = comm.next_slot()
            comm.slot_buffer(slot, rows, t.hidden).copy_(h)
            y, _ = comm.allreduce_norm(slot, rows, t.hidden, residual=res, weight=norm_w, eps=t.norm_eps,
                                       gemma=t.gemma_norm)
            return y
        return basic.rmsnorm(comm.all_reduce(h), norm_w, t.norm_eps, residual=res, gemma=t.gemma_norm)

    def _run_sublayer(self, sub, x, ctx, kv, states):
        if isinstance(sub, MoeLayer) and ctx.extras.get("ep") is not None:
            return sub.forward_a2a(x, ctx.extras["ep"])
        if isinstance(sub, MoeLayer) and sub.ep_size > 1 and ctx.comm is not None:
            return sub.forward_ep(x, ctx.comm)
        out = sub.forward(x, ctx, kv, states)
        if getattr(sub, "partial", False) and ctx.comm is not None:
            out = ctx.comm.all_reduce(out)
        return out

    def _hidden_states_hyper(self, ids: torch.Tensor, ctx: ForwardContext, kv, states=None):
        """Trunk with hyper-connections: the token's state is `hyper_streams` residual streams [T, hc * H]; a site's
        per-stream norm and gated mean stand where the pre-norm + residual add stand in the plain trunk.
        Reference: hibana/model/flashnext/model.py:42-77."""
        t = self.target
        hyper = self.embed_tokens(ids, ctx).repeat(1, t.hyper_streams)
        site = 0
        for bi, blk in enumerate(self.blocks):
            if bi in self.ple:
                hyper = basic.add(hyper, self.ple[bi].forward(hyper, ids, ctx, states))
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
        lg = gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
        if self.vocab_shard and comm is not None:
            lg = comm.all_gather_last(lg)
        return lg

    def greedy_tokens(self, normed: torch.Tensor, comm=None) -> torch.Tensor:
        """Greedy token per row; with a vocab-parallel head the ranks exchange one (value, id) pair per row."""
        from ..ops import sampling
        lg = gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
        if not (self.vocab_shard and comm is not None):
            return sampling.argmax(lg)
        idx, val = sampling.argmax_with_value(lg)
        if hasattr(comm, "pick_exchange"):
            return comm.pick_exchange(val, idx, self.target.tp_rank * self.vocab_shard)
        return sampling.argmax(comm.all_gather_last(lg))
