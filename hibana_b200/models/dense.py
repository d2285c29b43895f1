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

from .. import config as cfgmod
from ..engine.context import ForwardContext
from ..ops import attention, basic, gemm, nvfp4
from ..target import Target
from .linear import Linear, interleave_pairs, norm_linear


class DenseLayer:
    def __init__(self, t: Target, idx: int, gen: torch.Generator, device, std: float = 0.02, tp: int = 1,
                 rank: int = 0):
        """`t` is the unsharded target; with tp > 1 the full matrices are generated (same seed on every rank) and
        this rank's shard is cut out: q/k/v by head and gate/up by column (column-parallel), o_proj and down by
        input feature (row-parallel)."""
        h, d = t.hidden, t.head_dim
        fmt = "nvfp4" if t.weight_format == "nvfp4" else "bf16"

        def rnd(n, k):
            return torch.randn(n, k, generator=gen, dtype=torch.float32, device=gen.device) * std

        self.idx = idx
        self.input_norm = torch.ones(h, dtype=torch.bfloat16, device=device)
        self.post_norm = torch.ones(h, dtype=torch.bfloat16, device=device)
        wqkv, wo = rnd((t.q_heads + 2 * t.kv_heads) * d, h), rnd(h, t.q_heads * d)
        wgu, wd = interleave_pairs(rnd(t.ffn, h), rnd(t.ffn, h)), rnd(h, t.ffn)
        if tp == 1:
            self.qkv = Linear(wqkv, fmt, name=f"l{idx}.qkv").to(device)
            self.o = Linear(wo, fmt, name=f"l{idx}.o").to(device)
            self.gate_up = Linear(wgu, fmt, name=f"l{idx}.gate_up").to(device)
            self.down = Linear(wd, fmt, name=f"l{idx}.down").to(device)
            return
        hq, hkv = t.q_heads // tp, max(t.kv_heads // tp, 1)
        kv0 = (rank * t.kv_heads) // tp            # kv heads replicate when there are fewer than ranks
        qrows = torch.arange(rank * hq * d, (rank + 1) * hq * d)
        krows = t.q_heads * d + torch.arange(kv0 * d, (kv0 + hkv) * d)
        vrows = (t.q_heads + t.kv_heads) * d + torch.arange(kv0 * d, (kv0 + hkv) * d)
        f = t.ffn // tp
        # index tensors select rows; the quantised full matrix is sliced so shards are bitwise slices
        sel = torch.cat((qrows, krows, vrows)).to(wqkv.device)
        self.qkv = _shard(wqkv, fmt, rows=sel, name=f"l{idx}.qkv").to(device)
        self.o = _shard(wo, fmt, cols=slice(rank * hq * d, (rank + 1) * hq * d), name=f"l{idx}.o").to(device)
        self.gate_up = _shard(wgu, fmt, rows=slice(2 * rank * f, 2 * (rank + 1) * f), name=f"l{idx}.gate_up").to(device)
        self.down = _shard(wd, fmt, cols=slice(rank * f, (rank + 1) * f), name=f"l{idx}.down").to(device)

    def linears(self):
        return [self.qkv, self.o, self.gate_up, self.down]


def _shard(w, fmt, rows=None, cols=None, name=""):
    return Linear.sharded(w, fmt, rows=rows, cols=cols, name=name)


class DenseModel:
    """Random-init (N(0, 0.02), seeded) dense decoder. `forward` returns the final hidden rows to sample from.

    `target` is this rank's (sharded) geometry; `full` the unsharded one the weights are generated from."""

    def __init__(self, t: Target, device="cpu", seed: int = 0, init_device=None, *, full: Optional[Target] = None):
        self.target = t
        full = full or t
        tp, rank = t.tp_size, t.tp_rank
        self.device = torch.device(device)
        init_device = self.device if init_device is None else torch.device(init_device)
        gen = torch.Generator(device=init_device)
        gen.manual_seed(seed)
        self.embed = (torch.randn(full.vocab, full.hidden, generator=gen, dtype=torch.float32, device=init_device)
                      * 0.02).to(torch.bfloat16).to(self.device)
        self.layers = [DenseLayer(full, i, gen, self.device, tp=tp, rank=rank) for i in range(len(full.layers))]
        self.final_norm = torch.ones(full.hidden, dtype=torch.bfloat16, device=self.device)
        head = self.embed if full.tie_embeddings else (
            torch.randn(full.vocab, full.hidden, generator=gen, dtype=torch.float32, device=init_device) * 0.02
        ).to(torch.bfloat16).to(self.device)
        self.vocab_shard = full.vocab // tp if tp > 1 and full.vocab % tp == 0 else 0
        # vocab-parallel head: each rank scores vocab/tp tokens (reference: hibana/model/qwen38.py:181-182)
        self.lm_head = head[rank * self.vocab_shard:(rank + 1) * self.vocab_shard].contiguous() \
            if self.vocab_shard else head
        self.inv_freq = basic.rope_inv_freq(t.rot_dim, t.rope_theta, device=self.device) if t.rot_dim else \
            torch.zeros(1, device=self.device)
        self.scale = 1.0 / math.sqrt(t.head_dim)
        self.kv_layers = len(self.layers)

    @classmethod
    def sharded(cls, full: Target, tp: int, rank: int, device, seed: int = 0, init_device=None) -> "DenseModel":
        return cls(full.shard(tp, rank), device, seed, init_device, full=full)

    # ---- bookkeeping
    def linears(self):
        return [lin for layer in self.layers for lin in layer.linears()]

    def attach_w3(self) -> int:
        """3-bit decode copies of every projection (settings `w3`): decode and verify steps stream 4 bits per weight,
        prefill keeps the NVFP4 matrices. Returns the bytes the copies add."""
        added = 0
        for lin in self.linears():
            lin.attach_w3()
            added += lin.w3.nbytes()
        return added

    def weight_bytes(self) -> int:
        n = sum(lin.nbytes() for lin in self.linears()) + self.embed.numel() * 2
        if self.lm_head is not self.embed:
            n += self.lm_head.numel() * 2
        return n

    def calibrate(self, run_forward, comm=None) -> None:
        """Sets the static NVFP4 activation scales from one forward over sample tokens (random-init stand-in
        for the `input_scale` tensors a ModelOpt checkpoint ships). Ranks agree on the maximum."""
        lins = [lin for lin in self.linears() if lin.fmt == "nvfp4"]
        for lin in lins:
            lin.calibrating, lin.seen_amax = True, 0.0
        try:
            run_forward()
        finally:
            for lin in lins:
                lin.calibrating = False
        for lin in lins:
            amax = max(lin.seen_amax, 1e-3)
            if comm is not None:
                amax = comm.max_float(amax)
            lin.set_input_amax(amax * 1.5)

    # ---- forward
    def _reduce_norm_linear(self, h, slot, res, norm_w, lin, ctx, epilogue=gemm.EPI_STORE, requant=None):
        """lin(rmsnorm(allreduce(h) + res)). `h` is this rank's partial; with the fused path it already sits in
        heap slot `slot` and one kernel does all-reduce + add + norm + quant."""
        t = self.target
        comm = ctx.comm
        if comm is not None and slot is not None and not lin.calibrating:
            rows = h.shape[0]
            qs = lin.input_scale if lin.fmt == "nvfp4" and not lin.takes_w3(rows) else None
            y, xq = comm.allreduce_norm(slot, rows, t.hidden, residual=res, weight=norm_w, eps=t.norm_eps,
                                        quant_scale=qs, want_bf16=qs is None)
            return lin(xq if xq is not None else y, epilogue=epilogue, requant=requant)
        if comm is not None:
            h = comm.all_reduce(h)
        return norm_linear(h, res, norm_w, t.norm_eps, lin, epilogue=epilogue, requant=requant)

    def _row_parallel(self, lin, x, ctx):
        """Row-parallel projection; returns (partial, heap slot or None)."""
        comm = ctx.comm
        if comm is not None and comm.fits(x.shape[0] if not hasattr(x, "rows") else x.rows, self.target.hidden):
            slot = comm.next_slot()
            rows = x.shape[0] if not hasattr(x, "rows") else x.rows
            return lin(x, out=comm.slot_buffer(slot, rows, self.target.hidden)), slot
        return lin(x), None

    def forward_sp(self, ids: torch.Tensor, ctx: ForwardContext, kv) -> torch.Tensor:
        """Sequence-parallel prefill over the fused peer-memory chain: every row-parallel GEMM scatters its partial
        tiles to the rows' owner rank, the owner reduces + adds its residual shard + normalises + quantises and
        pushes the rows to every rank, and the next column-parallel GEMM starts each A tile as its rows arrive.
        The residual stream lives sharded by rows (rows_per_rank each)."""
        t = self.target
        comm = ctx.comm
        rows = ids.shape[0]
        rpr = rows // comm.world
        full = basic.embedding(ids, self.embed)
        res = full[comm.rank * rpr:(comm.rank + 1) * rpr].contiguous()
        qkv = norm_linear(full, None, self.layers[0].input_norm, t.norm_eps, self.layers[0].qkv, add_residual=False)
        y = None
        for i, layer in enumerate(self.layers):
            q = basic.rope_kv_write(qkv, ctx.positions, ctx.slots, self.inv_freq, kv.k[i], kv.v[i], t.q_heads,
                                    t.kv_heads, t.head_dim, rot=t.rot_dim, kv_scale=kv.kv_scale,
                                    table=basic.rope_table(ctx, self.inv_freq, t.rot_dim))
            att = attention.paged_attention(q, kv.k[i], kv.v[i], ctx.kv_indices, ctx.ctx_len, q_indptr=ctx.q_indptr,
                                            max_rows=ctx.max_rows, seq_rows=ctx.seq_rows, scale=self.scale,
                                            kv_scale=kv.kv_scale, splits=ctx.attn_splits,
                                            workspace=ctx.attn_workspace)
            comm.sp_gemm_scatter(layer.o, att.view(rows, -1))
            qs = layer.gate_up.input_scale if layer.gate_up.fmt == "nvfp4" else None
            x = comm.sp_reduce_norm_gather(rows, t.hidden, res, layer.post_norm, t.norm_eps, quant_scale=qs)
            act = comm.sp_gemm_gathered(layer.gate_up, x, epilogue=gemm.EPI_SILU_MUL)
            comm.sp_gemm_scatter(layer.down, act)
            if i + 1 < len(self.layers):
                nxt = self.layers[i + 1]
                qs = nxt.qkv.input_scale if nxt.qkv.fmt == "nvfp4" else None
                x = comm.sp_reduce_norm_gather(rows, t.hidden, res, nxt.input_norm, t.norm_eps, quant_scale=qs)
                qkv = comm.sp_gemm_gathered(nxt.qkv, x)
            else:
                y = comm.sp_reduce_norm_gather(rows, t.hidden, res, self.final_norm, t.norm_eps)
                # the bf16 gather buffer is complete on this rank only after every source's flag: a barrier orders it
                comm.barrier()
        return y.index_select(0, ctx.sample_rows) if ctx.sample_rows is not None else y.clone()

    def forward(self, ids: torch.Tensor, ctx: ForwardContext, kv) -> torch.Tensor:
        """ids int64 [T]; kv = KvPool. Returns normed hidden states of ctx.sample_rows (or of all rows)."""
        t = self.target
        if (ctx.comm is not None and getattr(ctx.comm, "sp_rows", 0) and ctx.mode == "prefill"
                and ctx.comm.sp_ok(ids.shape[0], t.hidden) and not self.layers[0].qkv.calibrating):
            return self.forward_sp(ids, ctx, kv)
        res = basic.embedding(ids, self.embed)
        if ctx.comm is None and self.layers[0].qkv.takes_gemv(ids.shape[0]) and self.layers[0].o.w3 is None:
            return self._forward_few_rows(res, ctx, kv)
        h: Optional[torch.Tensor] = None
        slot = None
        if ctx.comm is not None and hasattr(ctx.comm, "begin_forward"):
            ctx.comm.begin_forward(2 * len(self.layers))
        for i, layer in enumerate(self.layers):
            if h is None:
                qkv = norm_linear(res, None, layer.input_norm, t.norm_eps, layer.qkv, add_residual=False)
            else:
                qkv = self._reduce_norm_linear(h, slot, res, layer.input_norm, layer.qkv, ctx)
            q = basic.rope_kv_write(qkv, ctx.positions, ctx.slots, self.inv_freq, kv.k[i], kv.v[i], t.q_heads,
                                    t.kv_heads, t.head_dim, rot=t.rot_dim, kv_scale=kv.kv_scale,
                                    table=basic.rope_table(ctx, self.inv_freq, t.rot_dim))
            # decode-shaped steps hand NVFP4 activations from kernel to kernel: the attention kernel merges its KV
            # splits and quantises for o_proj, the gate/up GEMM requantises for down in its epilogue
            fuse = (cfgmod.current().fuse_epilogues and layer.o.fmt == "nvfp4" and not layer.o.calibrating
                    and q.shape[0] <= 128 and q.is_cuda and not layer.o.takes_w3(q.shape[0]))
            att = attention.paged_attention(q, kv.k[i], kv.v[i], ctx.kv_indices, ctx.ctx_len, q_indptr=ctx.q_indptr,
                                            max_rows=ctx.max_rows, seq_rows=ctx.seq_rows, scale=self.scale,
                                            kv_scale=kv.kv_scale, splits=ctx.attn_splits,
                                            workspace=ctx.attn_workspace,
                                            quant_scale=layer.o.input_scale if fuse else None)
            h, slot = self._row_parallel(layer.o, att if isinstance(att, nvfp4.Nvfp4Tensor)
                                         else att.view(att.shape[0], -1), ctx)
            # prefill-sized chunks requantise in the gate/up epilogue too (tokens on the 128-row side of the GEMM):
            # the bf16 activation [rows, intermediate] is never written
            fuse_mlp = fuse or (cfgmod.current().fuse_epilogues and q.is_cuda and layer.down.fmt == "nvfp4"
                                and not layer.down.calibrating and layer.gate_up.fmt == "nvfp4"
                                and gemm.requant_ok(q.shape[0], layer.gate_up.out_features))
            act = self._reduce_norm_linear(h, slot, res, layer.post_norm, layer.gate_up, ctx,
                                           epilogue=gemm.EPI_SILU_MUL,
                                           requant=layer.down.input_scale if fuse_mlp else None)
            h, slot = self._row_parallel(layer.down, act, ctx)
        comm = ctx.comm
        if comm is not None and slot is not None:
            y, _ = comm.allreduce_norm(slot, h.shape[0], t.hidden, residual=res, weight=self.final_norm,
                                       eps=t.norm_eps)
            return y.index_select(0, ctx.sample_rows) if ctx.sample_rows is not None else y
        if ctx.extras.get("want_hidden") is not None and comm is None:
            ctx.extras["hidden"] = basic.add(h, res)      # pre-norm hidden of every row: the drafters' feature
        if ctx.sample_rows is not None:
            h = h.index_select(0, ctx.sample_rows)
            res = res.index_select(0, ctx.sample_rows)
        if comm is not None:
            h = comm.all_reduce(h)
        return basic.rmsnorm(h, self.final_norm, t.norm_eps, residual=res)

    def _forward_few_rows(self, res: torch.Tensor, ctx: ForwardContext, kv) -> torch.Tensor:
        """Up to four rows on one GPU. The projections small enough for it (qkv and o at the 27B geometry) run the
        weight-streaming GEMV (ops/gemv.py) on bf16 activations, with the input norm in the qkv GEMV's prologue;
        every projection back into the hidden size adds its result to the residual stream in its own epilogue, in
        place, so no kernel of the layer exists only to add or normalise."""
        t = self.target
        rows = res.shape[0]
        for i, layer in enumerate(self.layers):
            qkv = norm_linear(res, None, layer.input_norm, t.norm_eps, layer.qkv, add_residual=False)
            q = basic.rope_kv_write(qkv, ctx.positions, ctx.slots, self.inv_freq, kv.k[i], kv.v[i], t.q_heads,
                                    t.kv_heads, t.head_dim, rot=t.rot_dim, kv_scale=kv.kv_scale,
                                    table=basic.rope_table(ctx, self.inv_freq, t.rot_dim))
            o_gemv = layer.o.takes_gemv(rows)
            att = attention.paged_attention(q, kv.k[i], kv.v[i], ctx.kv_indices, ctx.ctx_len, q_indptr=ctx.q_indptr,
                                            max_rows=ctx.max_rows, seq_rows=ctx.seq_rows, scale=self.scale,
                                            kv_scale=kv.kv_scale, splits=ctx.attn_splits,
                                            workspace=ctx.attn_workspace,
                                            quant_scale=None if o_gemv else layer.o.input_scale)
            layer.o(att if isinstance(att, nvfp4.Nvfp4Tensor) else att.view(rows, -1), epilogue=gemm.EPI_RESIDUAL,
                    residual=res, out=res)
            down_gemv = layer.down.takes_gemv(rows)
            act = norm_linear(res, None, layer.post_norm, t.norm_eps, layer.gate_up, epilogue=gemm.EPI_SILU_MUL,
                              add_residual=False, requant=None if down_gemv else layer.down.input_scale)
            layer.down(act, epilogue=gemm.EPI_RESIDUAL, residual=res, out=res)
        if ctx.extras.get("want_hidden") is not None:
            ctx.extras["hidden"] = res
        if ctx.sample_rows is not None:
            res = res.index_select(0, ctx.sample_rows)
        return basic.rmsnorm(res, self.final_norm, t.norm_eps)

    def greedy_tokens(self, normed: torch.Tensor, comm=None) -> torch.Tensor:
        """Greedy token of every row without materialising the full logits on any rank: with a vocab-parallel head
        each rank takes the maximum of its shard and the ranks exchange one (value, id) pair per row
        (`Communicator.pick_exchange`). Reference pattern: hibana/proposers/draft_head.py:229-285."""
        from ..ops import sampling
        lg = gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
        if not (self.vocab_shard and comm is not None):
            return sampling.argmax(lg)
        idx, val = sampling.argmax_with_value(lg)
        if hasattr(comm, "pick_exchange"):
            return comm.pick_exchange(val, idx, self.target.tp_rank * self.vocab_shard)
        return sampling.argmax(comm.all_gather_last(lg))

    def logits(self, normed: torch.Tensor, comm=None) -> torch.Tensor:
        lg = gemm.linear_bf16(normed, self.lm_head, epilogue=gemm.EPI_STORE_F32)
        if self.vocab_shard and comm is not None:
            lg = comm.all_gather_last(lg)
        return lg
