"""Bolt-class family: Nemotron geometry with heterogeneous MoE blocks and GGML-encoded weights served in place.

The published model ships its matrices as GGML blocks (routed experts IQ2_XXS / IQ2_XS at 2.06 / 2.31 bits per
weight, everything else Q8_0). Here they stay in those bytes on the device: `GgmlLinear` is the dense projection
(ops/ggml.py `PackedLinear` behind the interface the layer library calls) and `BoltMoeLayer` the latent MoE block
whose expert count and width come from the block's own spec (`Target.block`), with the (token, expert) pairs of a
decode step running as one grouped decode-fused launch per projection. Mamba-2, attention, the engine, caches and
speculation (LiLiCorr drafter, models/lilicorr.py) are the shared ones. Random-init weights: Q8_0 projections are
quantised from N(0, 0.02); IQ2 experts are random legal blocks over a synthetic lattice table unless the checkpoint's
tables are given (`Init.grids`), because the real tables are part of the file format and ship with the checkpoint.
Reference: hibana/model/bolt/model.py:33-251, hibana/model/bolt/linear.py:1-159, hibana/model/bolt/config.py.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..ops import basic, gemm, moe
from ..ops.ggml import PackedExperts, PackedLinear, random_blocks
from ..target import Target
from ..weights import ggml as fmt


class GgmlLinear(PackedLinear):
    """`PackedLinear` with the call signature of models/linear.py `Linear` (plain store epilogue only)."""
    calibrating = False

    @classmethod
    def from_weight(cls, w: torch.Tensor, name: str = "") -> "GgmlLinear":
        n, k = w.shape
        raw = torch.from_numpy(fmt.quantize_q8_0(w.float().cpu().numpy()))
        return cls(raw, fmt.T_Q8_0, n, k, None, name=name)

    def __call__(self, x, *, epilogue: int = gemm.EPI_STORE, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, requant=None, relu2: bool = False):
        if epilogue != gemm.EPI_STORE or requant is not None:
            raise NotImplementedError("GGML-packed projections have the plain epilogue")
        y = PackedLinear.__call__(self, x, relu2=relu2)
        if residual is not None:
            y = basic.add(y, residual)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def dequantized(self) -> torch.Tensor:
        return self.dequantize().float()


def synthetic_grid(entries: int, seed: int = 0) -> torch.Tensor:
    """A stand-in lattice table (magnitudes from the format's alphabet {8, 25, 43}) for random-init experts."""
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.choice(np.array([8, 25, 43], dtype=np.uint8), size=(entries, 8)))


class BoltMoeLayer:
    """Latent MoE block of the Bolt family: sigmoid router with selection bias, `t.experts` routed experts of width
    `t.expert_ffn` acting on the `t.latent`-wide projection (squared ReLU), a shared expert on the hidden state."""

    def __init__(self, t: Target, init, name: str, ep_rank: int = 0, ep_size: int = 1):
        """Tensor parallel (`ep_size` = the ranks, activations replicated): this rank keeps the experts
        [ep_rank * E / ep_size, ...) as block bytes of the full stacks and a column / row share of the shared
        expert; its output is a partial sum (`partial`: the block's all-reduce adds the ranks), the projection back
        from the latent being linear. A shared expert too narrow to split into whole Q8_0 blocks stays whole and only
        rank 0 adds it."""
        from .layers import MlpLayer
        self.t, self.ep_size, self.tp = t, ep_size, init.tp
        self.partial = ep_size > 1
        dev = init.device
        self.router = init.linear(t.experts, t.hidden, "bf16", name + ".router")
        self.sel_bias = torch.zeros(t.experts, device=dev)
        grids = getattr(init, "grids", None) or {}
        gx = grids.get("iq2_xxs", synthetic_grid(256, 1))
        gs = grids.get("iq2_xs", synthetic_grid(512, 2))
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=init.gen, device=init.gen_device))
        width = t.latent or t.hidden
        # block scales chosen so that activations keep the magnitude N(0, 0.02) matrices would give
        fc1 = PackedLinear(random_blocks("iq2_xxs", t.experts * t.expert_ffn, width, seed, scale=0.002).to(dev),
                           "iq2_xxs", t.experts * t.expert_ffn, width, gx, name + ".fc1")
        fc2 = PackedLinear(random_blocks("iq2_xs", t.experts * width, t.expert_ffn, seed + 1, scale=0.002).to(dev),
                           "iq2_xs", t.experts * width, t.expert_ffn, gs, name + ".fc2")
        self.experts = PackedExperts(fc1, fc2, t.experts)
        per = t.experts // ep_size
        self.e_lo = ep_rank * per
        if ep_size > 1:
            # every rank draws every expert (one seeded stream for every layout) and keeps its range
            if t.experts % ep_size:
                raise ValueError(f"{t.experts} experts do not divide over {ep_size} ranks")
            self.experts = self.experts.slice(self.e_lo, per)
        f = getattr(init, "full", None) or t
        shared_init, self.shared_owner = init, True
        if init.tp > 1 and t.shared_ffn and ((f.shared_ffn // init.tp) % 32 or f.shared_ffn % init.tp):
            import copy
            shared_init = copy.copy(init)          # same seeded stream, no sharding
            shared_init.tp, shared_init.rank = 1, 0
            self.shared_owner = init.rank == 0
        self.shared = (MlpLayer(t, shared_init, name + ".shared", width=f.shared_ffn, act="relu2")
                       if t.shared_ffn else None)
        self.fc1_latent = init.linear(t.latent, t.hidden, "q8_0", name + ".fc1_latent") if t.latent else None
        self.fc2_latent = init.linear(t.hidden, t.latent, "q8_0", name + ".fc2_latent") if t.latent else None

    def linears(self):
        out = [self.router]
        if self.shared is not None:
            out += self.shared.linears()
        return out + [l for l in (self.fc1_latent, self.fc2_latent) if l is not None]

    def forward(self, x, ctx=None, kv=None, states=None) -> torch.Tensor:
        t = self.t
        from ..utils import streams
        from .layers import overlap_ok
        # decode-sized on one GPU: the latent projection and the shared expert run on a side stream beside the router
        # and the routed experts (utils/streams.py); otherwise everything is one chain
        with streams.Branch(x, enabled=overlap_ok(x, ctx)) as br:
            inp = self.fc1_latent(x) if t.latent else x
            lat_ready = br.mark()
            shared = self.shared.forward(x) if self.shared is not None and self.shared_owner else None
        logits = gemm.linear_bf16(x, self.router.weight, epilogue=gemm.EPI_STORE_F32)
        ids, w = moe.route(logits, t.top_k, sigmoid=True, sel_bias=self.sel_bias, renorm=True, scale=t.router_scale)
        br.wait(lat_ready, inp if t.latent else None)
        y = self.experts.forward(inp, ids, w, id_base=self.e_lo)
        out = self.fc2_latent(y) if t.latent else y
        br.join(shared)
        return basic.add(out, shared) if shared is not None else out

    def weight_bytes(self) -> int:
        return self.experts.fc1.nbytes() + self.experts.fc2.nbytes()
