"""Dense GQA decoder (27B-class): pre-norm attention + SwiGLU MLP, NVFP4 or bf16 projections.

Per layer and forward: fused add+RMSNorm+quant -> qkv GEMM -> RoPE + KV-pool write -> paged attention ->
o_proj GEMM -> fused add+RMSNorm+quant -> gate_up GEMM with SiLU-mul epilogue -> down GEMM. With tensor
parallelism the o_proj / down partial sums are joined by the communicator (fused all-reduce + residual +
norm when available). Layer structure follows the reference's decoder layer (hibana/model/qwen38.py:53-78,
hibana/model/mlp.py:26-48) on the dense geometry of the benchmark configuration.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..engine.context import ForwardContext
from ..ops import attention, basic, gemm, nvfp4
from ..target import Target
from .linear import Linear, interleave_pairs, norm_linear


class DenseLayer:
    def __init__(self, t: Target, idx: int, gen: torch.Generator, device, std: float = 0.02):
        h, d = t.hidden, t.head_dim
        fmt = "nvfp4" if t.weight_format == "nvfp4" else "bf16"

        def rnd(n, k):
            return torch.randn(n, k, generator=gen, dtype=torch.float32, device=gen.device) * std

        self.idx = idx
        self.input_norm = torch.ones(h, dtype=torch.bfloat16, device=device)
        self.post_norm = torch.ones(h, dtype=torch.bfloat16, device=device)
        self.qkv = Linear(rnd((t.q_heads + 2 * t.kv_heads) * d, h), fmt, name=f"l{idx}.qkv").to(device)
        self.o = Linear(rnd(h, t.q_heads * d), fmt, name=f"l{idx}.o").to(device)
        self.gate_up = Linear(interleave_pairs(rnd(t.ffn, h), rnd(t.ffn, h)), fmt, name=f"l{idx}.gate_up").to(device)
        self.down = Linear(rnd(h, t.ffn), fmt, name=f"l{idx}.down").to(device)

    def linears(self):
        return [self.qkv, self.o, self.gate_up, self.down]


class DenseModel:
    """Random-init (N(0, 0.02), seeded) dense decoder. `forward` returns the final hidden rows to sample from."""

    def __init__(self, t: Target, device="cpu", seed: int = 0, init_device=None):
        self.target = t
        self.device = torch.device(device)
        init_device = self.device if init_device is None else torch.device(init_device)
        gen = torch.Generator(device=init_device)
        gen.manual_seed(seed)
        self.embed = (torch.randn(t.vocab, t.hidden, generator=gen, dtype=torch.float32, device=init_device)
                      * 0.02).to(torch.bfloat16).to(self.device)
        self.layers = [DenseLayer(t, i, gen, self.device) for i in range(len(t.layers))]
        self.final_norm = torch.ones(t.hidden, dtype=torch.bfloat16, device=self.device)
        self.lm_head = self.embed if t.tie_embeddings else (
            torch.randn(t.vocab, t.hidden, generator=gen, dtype=torch.float32, device=init_device) * 0.02
        ).to(torch.bfloat16).to(self.device)
        self.inv_freq = basic.rope_inv_freq(t.rot_dim, t.rope_theta, device=self.device) if t.rot_dim else \
            torch.zeros(1, device=self.device)
        self.scale = 1.0 / math.sqrt(t.head_dim)
        self.kv_layers = len(self.layers)

    # ---- bookkeeping
    def linears(self):
        return [lin for layer in self.layers for lin in layer.linears()]

    def weight_bytes(self) -> int:
        n = sum(lin.nbytes() for lin in self.linears()) + self.embed.numel() * 2
        if self.lm_head is not self.embed:
            n += self.lm_head.numel() * 2
        return n

    def calibrate(self, run_forward) -> None:
        """Sets the static NVFP4 activation scales from one forward over sample tokens (random-init stand-in
        for the `input_scale` tensors a ModelOpt checkpoint ships)."""
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
    def forward(self, ids: torch.Tensor, ctx: ForwardContext, kv) -> torch.Tensor:
        """ids int64 [T]; kv = KvPool. Returns normed hidden states of ctx.sample_rows (or of all rows)."""
        t = self.target
        res = basic.embedding(ids, self.embed)
        h: Optional[torch.Tensor] = None
        for i, layer in enumerate(self.layers):
            if h is None:
                qkv = norm_linear(res, None, layer.input_norm, t.norm_eps, layer.qkv, add_residual=False)
            else:
                qkv = norm_linear(h, res, layer.input_norm, t.norm_eps, layer.qkv)
            q = basic.rope_kv_write(qkv, ctx.positions, ctx.slots, self.inv_freq, kv.k[i], kv.v[i], t.q_heads,
                                    t.kv_heads, t.head_dim, rot=t.rot_dim, kv_scale=kv.kv_scale)
            att = attention.paged_attention(q, kv.k[i], kv.v[i], ctx.kv_indices, ctx.ctx_len, q_indptr=ctx.q_indptr,
                                            max_rows=ctx.max_rows, seq_rows=ctx.seq_rows, scale=self.scale, kv_scale=kv.kv_scale,
                                            splits=ctx.attn_splits, workspace=ctx.attn_workspace)
            h = layer.o(att.view(att.shape[0], -1))
            if ctx.comm is not None:
                h = ctx.comm.all_reduce(h)
            act = norm_linear(h, res, layer.post_norm, t.norm_eps, layer.gate_up, epilogue=gemm.EPI_SILU_MUL)
            h = layer.down(act)
            if ctx.comm is not None:
                h = ctx.comm.all_reduce(h)
        if ctx.sample_rows is not None:
            h = h.index_select(0, ctx.sample_rows)
            res = res.index_select(0, ctx.sample_rows)
        return basic.rmsnorm(h, self.final_norm, t.norm_eps, residual=res)

    def logits(self, normed: torch.Tensor) -> torch.Tensor:
        return gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
