"""Layer library of the hybrid model families: attention (plain / gated-output), Mamba-2, gated delta rule,
SwiGLU MLP, MoE with shared expert, latent MoE. Every layer holds its weights and a `forward(x, ctx, caches)`
that takes the normed input rows and returns this rank's output rows (a partial sum under tensor parallelism).

Reference: hibana/model/attention.py:69-126, hibana/model/gdn.py:41-301, hibana/model/nemotron/mamba.py:23-86,
hibana/model/mlp.py:26-48, hibana/model/flashnext/moe.py:68-192, hibana/model/nemotron/moe.py:349-566.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import config as cfgmod
from ..engine.context import ForwardContext
from ..ops import attention, basic, gemm, moe, recurrent
from ..target import ATTN, GATED_ATTN, GDN, LATENT_MOE, MAMBA2, MLP, MOE, NONE, Target
from ..utils import streams
from .linear import Linear, interleave_pairs


class Init:
    """Seeded weight factory (N(0, std) matrices) shared by all layers of a model."""

    def __init__(self, seed: int, device, init_device=None, std: float = 0.02, tp: int = 1, rank: int = 0,
                 full: Optional[Target] = None):
        """`tp` / `rank`: tensor-parallel shard to keep. Every rank draws the FULL matrices from the same seeded
        stream (so the unsharded model is the same on every rank and for every tp) and keeps its rows / columns;
        `full` is the unsharded target the shapes come from."""
        self.tp, self.rank, self.full = tp, rank, full
        self.device = torch.device(device)
        self.gen_device = torch.device(init_device) if init_device is not None else self.device
        self.gen = torch.Generator(device=self.gen_device)
        self.gen.manual_seed(seed)
        self.std = std

    def normal(self, *shape, std: Optional[float] = None) -> torch.Tensor:
        return torch.randn(*shape, generator=self.gen, dtype=torch.float32, device=self.gen_device) * (std or self.std)

    def uniform(self, *shape, lo: float = 0.0, hi: float = 1.0) -> torch.Tensor:
        return torch.rand(*shape, generator=self.gen, dtype=torch.float32, device=self.gen_device) * (hi - lo) + lo

    def linear(self, n: int, k: int, fmt: str, name: str = "", rows=None, cols=None) -> Linear:
        """[n, k] projection; `rows` / `cols` (slice or index tensor) keep a tensor-parallel shard that is bitwise a
        slice of the quantised full matrix. fmt "q8_0": GGML Q8_0 blocks served in place (models/bolt.py)."""
        w = self.normal(n, k)
        if fmt == "q8_0":
            from .bolt import GgmlLinear
            lin = GgmlLinear.from_weight(w, name=name)
            if rows is not None or cols is not None:
                lin = lin.shard(rows=rows, cols=cols)      # block bytes of the full matrix: nothing requantised
            return lin.to(self.device)
        if rows is None and cols is None:
            return Linear(w, fmt, name=name).to(self.device)
        if isinstance(rows, torch.Tensor):
            rows = rows.to(w.device)
        return Linear.sharded(w, fmt, rows=rows, cols=cols, name=name).to(self.device)

    def span(self, per_rank: int) -> slice:
        """This rank's contiguous range of `per_rank` items."""
        return slice(self.rank * per_rank, (self.rank + 1) * per_rank)

    def rows_of(self, *ranges) -> Optional[torch.Tensor]:
        """Index tensor over several (offset, start, length) row ranges (None without tensor parallelism)."""
        if self.tp == 1:
            return None
        return torch.cat([torch.arange(off + lo, off + lo + n) for off, lo, n in ranges])

    def take(self, x: torch.Tensor, idx) -> torch.Tensor:
        if idx is None:
            return x
        return x[idx.to(x.device) if isinstance(idx, torch.Tensor) else idx]

    def ones(self, n: int, gemma: bool = False) -> torch.Tensor:
        return (torch.zeros if gemma else torch.ones)(n, dtype=torch.bfloat16, device=self.device)


def _fmt(t: Target) -> str:
    return "nvfp4" if t.weight_format == "nvfp4" else "q8_0" if t.weight_format == "ggml" else "bf16"


class AttentionLayer:
    def __init__(self, t: Target, init: Init, kv_index: int, gated: bool, name: str):
        d = t.head_dim
        self.t, self.kv_index, self.gated = t, kv_index, gated
        f = init.full or t                      # unsharded geometry (t holds this rank's head counts)
        gq = 2 if gated else 1
        qw = f.q_heads * d * gq
        # tensor parallel: q (and gate) rows by head, k / v rows by kv head (replicated when kv heads < ranks),
        # o_proj by input feature; the output is then a partial sum
        kv0 = (init.rank * f.kv_heads) // init.tp
        rows = init.rows_of((0, init.rank * t.q_heads * d * gq, t.q_heads * d * gq),
                            (qw, kv0 * d, t.kv_heads * d), (qw + f.kv_heads * d, kv0 * d, t.kv_heads * d))
        self.qkv = init.linear(qw + 2 * f.kv_heads * d, t.hidden, _fmt(t), name + ".qkv", rows=rows)
        self.o = init.linear(t.hidden, f.q_heads * d, _fmt(t), name + ".o",
                             cols=init.span(t.q_heads * d) if init.tp > 1 else None)
        # the projection that reads the normed rows (the norm can quantise straight into its format) and whether
        # anything else of the layer still needs them in bf16
        self.first, self.needs_x = self.qkv, t.qsa_ratio > 0       # the indexer projects the normed rows too
        self.partial = init.tp > 1
        self.q_norm = init.ones(d, t.gemma_norm) if t.qk_norm else None
        self.k_norm = init.ones(d, t.gemma_norm) if t.qk_norm else None
        self.inv_freq = basic.rope_inv_freq(max(t.rot_dim, 2), t.rope_theta, device=init.device)
        self.scale = 1.0 / math.sqrt(d)
        # sparse-attention indexer (long contexts): 128-wide index queries / keys beside the real ones
        self.indexer = None
        if t.qsa_ratio:
            from .qsa import QD, QsaIndexer
            self.idx_q = init.linear(t.qsa_heads * QD, t.hidden, "bf16", name + ".idx_q")
            self.idx_k = init.linear(QD, t.hidden, "bf16", name + ".idx_k")
            self.indexer = QsaIndexer(t.qsa_ratio, t.qsa_budget, t.qsa_heads, rot=64, eps=t.norm_eps,
                                      theta=t.rope_theta, device=init.device)

    def linears(self):
        return [self.qkv, self.o] + ([self.idx_q, self.idx_k] if self.indexer is not None else [])

    def _sparse(self, x, q, ctx: ForwardContext, kv) -> torch.Tensor:
        """Attention through the indexer: every query row attends to the `qsa_budget` best-scoring KV tokens (whole
        groups of `qsa_ratio`, chosen by its index queries against the groups' compressed index keys) and the tail
        of its own group. With no more groups than the budget holds the result is dense causal attention."""
        from .qsa import QD, _rope
        t, ix, i = self.t, self.indexer, self.kv_index
        rows = x.shape[0]
        kv.idx_raw[i].index_copy_(0, ctx.slots.long(), self.idx_k(x))
        if ctx.q_indptr is None:
            per_seq = torch.ones_like(ctx.ctx_len)
            row_seq = ctx.seq_rows if ctx.seq_rows is not None else torch.arange(rows, dtype=torch.int32, device=x.device)
        else:
            per_seq = ctx.q_indptr[1:] - ctx.q_indptr[:-1]
            seqs = ctx.seq_rows if ctx.seq_rows is not None else torch.arange(per_seq.numel(), dtype=torch.int32,
                                                                              device=x.device)
            counts = ctx.seq_starts_host if ctx.seq_starts_host is not None else per_seq.tolist()
            row_seq = torch.repeat_interleave(seqs, torch.as_tensor(counts, device=x.device), output_size=rows)
        first = torch.div(ctx.ctx_len - per_seq, ix.ratio, rounding_mode="floor").int()
        count = torch.div(ctx.ctx_len, ix.ratio, rounding_mode="floor").int() - first
        ix.compress(kv.idx_raw[i], kv.idx_key[i], ctx.kv_indices, ctx.seq_rows, first, count,
                    max_total=rows // ix.ratio + per_seq.numel())
        qi = _rope(self.idx_q(x).view(rows, ix.heads, QD), ctx.positions, ix.rot, ix.inv_freq).to(torch.bfloat16)
        max_pos = int(ctx.extras.get("qsa_max_pos") or ctx.max_ctx_host or ctx.kv_indices.shape[1]) - 1
        sel, sel_len = ix.select(qi.contiguous(), kv.idx_key[i], ctx.kv_indices, row_seq.int().contiguous(),
                                 ctx.positions.int().contiguous(), max_pos)
        return ix.sparse_attention(q, kv.k[i], kv.v[i], sel, sel_len, scale=self.scale, kv_scale=kv.kv_scale)

    def forward(self, x, ctx: ForwardContext, kv, states, xq=None) -> torch.Tensor:
        t = self.t
        qkv = self.qkv(x if xq is None else xq)
        i = self.kv_index
        q = basic.rope_kv_write(qkv, ctx.positions, ctx.slots, self.inv_freq, kv.k[i], kv.v[i], t.q_heads,
                                t.kv_heads, t.head_dim, rot=t.rot_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                                eps=t.norm_eps, gemma_norm=t.gemma_norm, kv_scale=kv.kv_scale, q_gate=self.gated,
                                table=basic.rope_table(ctx, self.inv_freq, t.rot_dim))
        if self.indexer is not None and ctx.extras.get("qsa") and kv.idx_raw:
            att = self._sparse(x, q, ctx, kv)
        else:
            att = attention.paged_attention(q, kv.k[i], kv.v[i], ctx.kv_indices, ctx.ctx_len, q_indptr=ctx.q_indptr,
                                            max_rows=ctx.max_rows, seq_rows=ctx.seq_rows, scale=self.scale,
                                            kv_scale=kv.kv_scale, splits=ctx.attn_splits,
                                            workspace=ctx.attn_workspace)
        att = att.view(att.shape[0], -1)
        if self.gated:
            d = t.head_dim
            gate = qkv[:, :t.q_heads * 2 * d].view(-1, t.q_heads, 2 * d)[..., d:].reshape(att.shape[0], -1)
            att = basic.act_mul(att, basic.ACT_SIGMOID_GATE, gate.contiguous())
        return self.o(att)


class MambaLayer:
    def __init__(self, t: Target, init: Init, state_index: int, name: str):
        self.t, self.state_index = t, state_index
        f = init.full or t
        inner, gn = t.mamba_inner, t.mamba_groups * t.mamba_state          # this rank's widths
        finner, fgn = f.mamba_inner, f.mamba_groups * f.mamba_state
        # tensor parallel: heads split by rank, B / C groups follow their heads (a group is replicated when there
        # are fewer groups than ranks); rows of in_proj are z | x | B | C | dt, conv channels x | B | C
        g0 = (init.rank * f.mamba_groups) // init.tp
        sel = init.rows_of((0, init.rank * inner, inner), (finner, init.rank * inner, inner),
                           (2 * finner, g0 * t.mamba_state, gn), (2 * finner + fgn, g0 * t.mamba_state, gn),
                           (2 * finner + 2 * fgn, init.rank * t.mamba_heads, t.mamba_heads))
        csel = init.rows_of((0, init.rank * inner, inner), (finner, g0 * t.mamba_state, gn),
                            (finner + fgn, g0 * t.mamba_state, gn))
        hsel = init.span(t.mamba_heads) if init.tp > 1 else None
        self.in_proj = init.linear(2 * finner + 2 * fgn + f.mamba_heads, t.hidden, _fmt(t), name + ".in_proj", rows=sel)
        self.out_proj = init.linear(t.hidden, finner, _fmt(t), name + ".out_proj",
                                    cols=init.span(inner) if init.tp > 1 else None)
        self.conv_w = init.take(init.normal(f.mamba_conv_dim, t.conv_width, std=0.2), csel).to(torch.bfloat16).to(init.device)
        self.conv_b = init.take(init.normal(f.mamba_conv_dim, std=0.02), csel).to(torch.bfloat16).to(init.device)
        self.a_log = init.take(torch.log(init.uniform(f.mamba_heads, lo=1.0, hi=16.0)), hsel).to(init.device)
        dt = torch.exp(init.uniform(f.mamba_heads) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        self.dt_bias = init.take(dt + torch.log(-torch.expm1(-dt)), hsel).to(init.device)       # inverse softplus
        self.d_skip = torch.ones(t.mamba_heads, device=init.device)
        self.norm_w = init.ones(inner)
        # the projection that reads the normed rows (the norm can quantise straight into its format) and whether
        # anything else of the layer still needs them in bf16
        self.first, self.needs_x = self.in_proj, False
        self.partial = init.tp > 1

    def linears(self):
        return [self.in_proj, self.out_proj]

    def forward(self, x, ctx: ForwardContext, kv, states, xq=None) -> torch.Tensor:
        t = self.t
        inner, gn = t.mamba_inner, t.mamba_groups * t.mamba_state
        zxbcdt = self.in_proj(x if xq is None else xq)
        z = zxbcdt[:, :inner]
        xbc = zxbcdt[:, inner:2 * inner + 2 * gn]
        dt = zxbcdt[:, 2 * inner + 2 * gn:]
        li = self.state_index
        so = ctx.extras.get("state_out", ctx.state_slots)
        if "ring" in ctx.extras:      # verify: log the recurrence inputs so the accepted prefix can be replayed
            ctx.extras["ring"].append((self, (xbc, dt)))
        xbc = recurrent.conv1d(xbc, self.conv_w, self.conv_b, states.conv[li], ctx.state_slots, so,
                               q_indptr=ctx.q_indptr, has_init=ctx.has_initial_state, silu=True,
                               max_rows=ctx.max_rows if ctx.q_indptr is not None else 0)
        if getattr(states, "window", 0):
            y = self._scan_window(xbc, dt, states, ctx.state_slots, ctx.q_indptr, ctx.has_initial_state,
                                  ctx.seq_starts_host, commit="state_out" not in ctx.extras)
        else:
            y = recurrent.mamba2_scan(xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:], dt, self.a_log,
                                      self.dt_bias, self.d_skip, states.ssm[li], ctx.state_slots, so,
                                      heads=t.mamba_heads, groups=t.mamba_groups, head_dim=t.mamba_head_dim,
                                      d_state=t.mamba_state, q_indptr=ctx.q_indptr, has_init=ctx.has_initial_state,
                                      state_scale=states.ssm_scale[li] if getattr(states, "ssm_scale", None) is not None
                                      else None, sr_seed=ctx.extras.get("sr_seed", 0), host_rows=ctx.seq_starts_host)
        if self.out_proj.fmt == "nvfp4" and not self.out_proj.calibrating and not self.out_proj.takes_w3(y.shape[0]):
            # the gated norm writes the output projection's NVFP4 input itself
            return self.out_proj(basic.gated_rmsnorm_quant(y, z, self.norm_w, t.norm_eps, inner // t.mamba_groups,
                                                           self.out_proj.input_scale))
        y = basic.gated_rmsnorm(y, z, self.norm_w, t.norm_eps, inner // t.mamba_groups)
        return self.out_proj(y)

    def _scan_window(self, xbc, dt, states, slots, q_indptr, has_init, host_rows, commit: bool) -> torch.Tensor:
        """The scan over the window-record state format (ops/ssm_window.py). Decode, verify and replay rows read the
        int8 boundary state and the committed-token records in place (a verify pass writes nothing); a prefill chunk
        runs the fp32 kernels on a temporary state expanded from the record and folds the result back."""
        from ..ops import ssm_window
        t = self.t
        inner, gn = t.mamba_inner, t.mamba_groups * t.mamba_state
        ws = states.window_state(self.state_index)
        xs, bm, cm = xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:]
        long_rows = host_rows is not None and q_indptr is not None and max(host_rows) > ssm_window.MAX_ROWS
        if not long_rows:
            return ssm_window.step(ws, xs, bm, cm, dt, self.a_log, self.dt_bias, self.d_skip, slots, q_indptr=q_indptr,
                                   has_init=has_init, commit=commit)
        b = slots.shape[0]
        dense = ssm_window.to_dense(ws, slots)
        if has_init is not None:
            dense = dense * has_init.to(dense.dtype).view(b, 1, 1, 1)
        tmp = torch.arange(b, dtype=torch.int32, device=slots.device)
        y = recurrent.mamba2_scan(xs, bm, cm, dt, self.a_log, self.dt_bias, self.d_skip, dense, tmp, tmp,
                                  heads=t.mamba_heads, groups=t.mamba_groups, head_dim=t.mamba_head_dim,
                                  d_state=t.mamba_state, q_indptr=q_indptr, host_rows=host_rows)
        if commit:
            ssm_window.from_dense(ws, slots, dense)
        return y

    def replay(self, saved, sel, q_indptr, slots, states) -> None:
        """Advances the committed state over the selected (accepted) rows of a verify block."""
        t = self.t
        inner, gn = t.mamba_inner, t.mamba_groups * t.mamba_state
        xbc, dt = saved[0].index_select(0, sel), saved[1].index_select(0, sel)
        li = self.state_index
        xbc = recurrent.conv1d(xbc, self.conv_w, self.conv_b, states.conv[li], slots, slots, q_indptr=q_indptr)
        if getattr(states, "window", 0):
            self._scan_window(xbc, dt, states, slots, q_indptr, None, None, commit=True)
            return
        recurrent.mamba2_scan(xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:], dt, self.a_log,
                              self.dt_bias, self.d_skip, states.ssm[li], slots, slots, heads=t.mamba_heads,
                              groups=t.mamba_groups, head_dim=t.mamba_head_dim, d_state=t.mamba_state,
                              q_indptr=q_indptr, state_scale=states.ssm_scale[li]
                              if getattr(states, "ssm_scale", None) is not None else None)


class GdnLayer:
    def __init__(self, t: Target, init: Init, state_index: int, name: str):
        self.t, self.state_index = t, state_index
        kd = t.gdn_head_dim
        f = init.full or t
        self.qk = t.gdn_k_heads * kd
        self.vd = t.gdn_v_heads * kd
        fqk, fvd = f.gdn_k_heads * kd, f.gdn_v_heads * kd
        # tensor parallel: key heads and their value heads split by rank; rows of in_qkvz are q | k | v | z
        r = init.rank
        sel = init.rows_of((0, r * self.qk, self.qk), (fqk, r * self.qk, self.qk), (2 * fqk, r * self.vd, self.vd),
                           (2 * fqk + fvd, r * self.vd, self.vd))
        csel = init.rows_of((0, r * self.qk, self.qk), (fqk, r * self.qk, self.qk), (2 * fqk, r * self.vd, self.vd))
        basel = init.rows_of((0, r * t.gdn_v_heads, t.gdn_v_heads), (f.gdn_v_heads, r * t.gdn_v_heads, t.gdn_v_heads))
        hsel = init.span(t.gdn_v_heads) if init.tp > 1 else None
        self.in_qkvz = init.linear(2 * fqk + 2 * fvd, t.hidden, _fmt(t), name + ".in_qkvz", rows=sel)
        self.in_ba = init.linear(2 * f.gdn_v_heads, t.hidden, "bf16", name + ".in_ba", rows=basel)
        self.out_proj = init.linear(t.hidden, fvd, _fmt(t), name + ".out_proj",
                                    cols=init.span(self.vd) if init.tp > 1 else None)
        self.conv_w = init.take(init.normal(f.gdn_conv_dim, t.conv_width, std=0.2), csel).to(torch.bfloat16).to(init.device)
        self.a_log = init.take(torch.log(init.uniform(f.gdn_v_heads, lo=1.0, hi=16.0)), hsel).to(init.device)
        self.dt_bias = init.take(init.normal(f.gdn_v_heads, std=0.5), hsel).to(init.device)
        self.norm_w = init.ones(kd, t.gemma_norm)
        self.norm_w_heads, self._norm_w_key = None, None          # norm_w repeated per head, rebuilt when it changes
        # the projection that reads the normed rows (the norm can quantise straight into its format) and whether
        # anything else of the layer still needs them in bf16
        self.first, self.needs_x = self.in_qkvz, True
        self.partial = init.tp > 1

    def linears(self):
        return [self.in_qkvz, self.in_ba, self.out_proj]

    def forward(self, x, ctx: ForwardContext, kv, states, xq=None) -> torch.Tensor:
        t = self.t
        kd = t.gdn_head_dim
        # the gate projection (quantise, GEMM, gate kernel) does not meet the q / k / v chain before the scan: at
        # decode sizes it runs on a side stream beside in_qkvz and the convolution (utils/streams.py)
        with streams.Branch(x, enabled=overlap_ok(x, ctx, comm_free=True)) as br:
            beta, g = basic.gdn_gates(self.in_ba(x), self.a_log, self.dt_bias)
        qkvz = self.in_qkvz(x if xq is None else xq)
        li = self.state_index
        so = ctx.extras.get("state_out", ctx.state_slots)
        if "ring" in ctx.extras:
            ctx.extras["ring"].append((self, (qkvz[:, :2 * self.qk + self.vd], g, beta)))
        qkv = recurrent.conv1d(qkvz[:, :2 * self.qk + self.vd], self.conv_w, None, states.conv[li], ctx.state_slots,
                               so, q_indptr=ctx.q_indptr, has_init=ctx.has_initial_state, silu=True,
                               max_rows=ctx.max_rows if ctx.q_indptr is not None else 0)
        z = qkvz[:, 2 * self.qk + self.vd:]
        br.join(beta, g)
        if getattr(states, "window", 0):
            o = self._scan_window(qkv, g, beta, states, ctx.state_slots, ctx.q_indptr, ctx.has_initial_state,
                                  ctx.seq_starts_host, commit="state_out" not in ctx.extras)
        else:
            o = recurrent.gdn_scan(qkv[:, :self.qk], qkv[:, self.qk:2 * self.qk], qkv[:, 2 * self.qk:], g, beta,
                                   states.ssm[li], ctx.state_slots, so, k_heads=t.gdn_k_heads, v_heads=t.gdn_v_heads,
                                   kdim=kd, vdim=kd, l2norm=True, q_indptr=ctx.q_indptr,
                                   has_init=ctx.has_initial_state, host_rows=ctx.seq_starts_host)
        rows = o.shape[0]
        # per-head RMSNorm of the output, then the SiLU gate (norm before gate)
        key = (id(self.norm_w), self.norm_w._version)
        if self._norm_w_key != key:
            self.norm_w_heads, self._norm_w_key = self.norm_w.repeat(t.gdn_v_heads), key
        w = self.norm_w_heads
        if self.out_proj.fmt == "nvfp4" and not self.out_proj.calibrating and not self.out_proj.takes_w3(rows):
            return self.out_proj(basic.gated_rmsnorm_quant(o, z, w, t.norm_eps, kd, self.out_proj.input_scale,
                                                           norm_first=True, gemma=t.gemma_norm))
        y = basic.gated_rmsnorm(o, z, w, t.norm_eps, kd, norm_first=True, gemma=t.gemma_norm)
        return self.out_proj(y.view(rows, -1))

    def _scan_window(self, qkv, g, beta, states, slots, q_indptr, has_init, host_rows, commit: bool) -> torch.Tensor:
        """The delta rule over the window-record state format (ops/ssm_window.py `step_delta`): decode, verify and
        replay rows in place (verify writes nothing); prefill chunks through a temporary fp32 state."""
        from ..ops import ssm_window
        t = self.t
        kd = t.gdn_head_dim
        ws = states.window_state(self.state_index)
        q, k, v = qkv[:, :self.qk], qkv[:, self.qk:2 * self.qk], qkv[:, 2 * self.qk:]
        long_rows = host_rows is not None and q_indptr is not None and max(host_rows) > ssm_window.MAX_ROWS
        if not long_rows:
            return ssm_window.step_delta(ws, q, k, v, g, beta, slots, l2norm=True, q_indptr=q_indptr, has_init=has_init,
                                         commit=commit)
        b = slots.shape[0]
        dense = ssm_window.to_dense(ws, slots)
        if has_init is not None:
            dense = dense * has_init.to(dense.dtype).view(b, 1, 1, 1)
        tmp = torch.arange(b, dtype=torch.int32, device=slots.device)
        o = recurrent.gdn_scan(q, k, v, g, beta, dense, tmp, tmp, k_heads=t.gdn_k_heads, v_heads=t.gdn_v_heads,
                               kdim=kd, vdim=kd, l2norm=True, q_indptr=q_indptr, host_rows=host_rows)
        if commit:
            ssm_window.from_dense(ws, slots, dense)
        return o

    def replay(self, saved, sel, q_indptr, slots, states) -> None:
        t = self.t
        kd = t.gdn_head_dim
        li = self.state_index
        qkv = recurrent.conv1d(saved[0].index_select(0, sel), self.conv_w, None, states.conv[li], slots, slots,
                               q_indptr=q_indptr)
        if getattr(states, "window", 0):
            self._scan_window(qkv, saved[1].index_select(0, sel).contiguous(),
                              saved[2].index_select(0, sel).contiguous(), states, slots, q_indptr, None, None, True)
            return
        recurrent.gdn_scan(qkv[:, :self.qk], qkv[:, self.qk:2 * self.qk], qkv[:, 2 * self.qk:],
                           saved[1].index_select(0, sel).contiguous(), saved[2].index_select(0, sel).contiguous(),
                           states.ssm[li], slots, slots, k_heads=t.gdn_k_heads, v_heads=t.gdn_v_heads, kdim=kd,
                           vdim=kd, l2norm=True, q_indptr=q_indptr)


class MlpLayer:
    def __init__(self, t: Target, init: Init, name: str, width: Optional[int] = None, act: str = "swiglu"):
        """`width` is the UNSHARDED intermediate size; with tensor parallelism this rank keeps width / tp columns of
        gate / up (rows of the stacked matrix) and the matching input features of down."""
        self.t, self.act = t, act
        width = width or (init.full or t).ffn
        local = width // init.tp
        if act == "swiglu":
            w = interleave_pairs(init.normal(width, t.hidden), init.normal(width, t.hidden))
            self.up = (Linear(w, _fmt(t), name=name + ".gate_up") if init.tp == 1 else
                       Linear.sharded(w, _fmt(t), rows=slice(2 * init.rank * local, 2 * (init.rank + 1) * local),
                                      name=name + ".gate_up")).to(init.device)
        else:
            self.up = init.linear(width, t.hidden, _fmt(t), name + ".up", rows=init.span(local) if init.tp > 1 else None)
        self.down = init.linear(t.hidden, width, _fmt(t), name + ".down", cols=init.span(local) if init.tp > 1 else None)
        # the projection that reads the normed rows (the norm can quantise straight into its format) and whether
        # anything else of the layer still needs them in bf16
        self.first, self.needs_x = self.up, False
        self.partial = init.tp > 1

    def linears(self):
        return [self.up, self.down]

    def forward(self, x, ctx=None, kv=None, states=None, xq=None) -> torch.Tensor:
        x = x if xq is None else xq
        if self.act == "swiglu":
            return self.down(self.up(x, epilogue=gemm.EPI_SILU_MUL))
        return self.down(basic.act_mul(self.up(x), basic.ACT_RELU2))


def overlap_ok(x: torch.Tensor, ctx, comm_free: bool = False) -> bool:
    """Side-stream branches inside a layer: CUDA tensors and decode-sized row counts. A branch that could reach the
    communicator needs `ctx.comm` to be absent (its kernels and heap slots are ordered on one stream); a branch of
    plain local launches (`comm_free`) may run beside a tensor-parallel layer too."""
    rows = cfgmod.current().overlap_rows
    if not x.is_cuda or not 0 < x.shape[0] <= rows:
        return False
    return comm_free or ctx is None or getattr(ctx, "comm", None) is None


class MoeLayer:
    """Routed experts (+ shared expert). With `latent` > 0 the experts act on a down-projected latent and the sum is
    projected back (Nemotron); the shared expert always acts on the hidden state."""

    def __init__(self, t: Target, init: Init, name: str, ep_rank: int = 0, ep_size: int = 1):
        self.t = t
        width = t.latent or t.hidden
        n1 = 2 * t.expert_ffn if t.moe_act == "swiglu" else t.expert_ffn
        self.router = init.linear(t.experts, t.hidden, "bf16", name + ".router")
        self.sel_bias = torch.zeros(t.experts, device=init.device) if t.router == "sigmoid" else None
        fc1 = init.normal(t.experts, n1, width)
        if t.moe_act == "swiglu":   # rows g0, u0, g1, u1, ... inside every expert
            fc1 = torch.stack((fc1[:, :t.expert_ffn], fc1[:, t.expert_ffn:]), dim=2).reshape(t.experts, n1, width)
        fc2 = init.normal(t.experts, width, t.expert_ffn)
        per = t.experts // ep_size
        self.e_lo, self.e_n = ep_rank * per, per
        # an expert-parallel rank draws every expert (one seeded stream for every layout) and keeps its range
        keep = slice(self.e_lo, self.e_lo + per)
        self.experts = moe.ExpertWeights.create(fc1[keep], fc2[keep], t.moe_act, _fmt(t)).to(init.device)
        del fc1, fc2
        f = init.full or t
        # under tensor parallelism the shared expert is column / row split like a dense MLP (its partial sum joins
        # the routed experts' partial sum before the one all-reduce of the layer) when a rank's share of its width is
        # a whole number of 64-feature K tiles; a narrower shared expert (640 wide over 8 ranks) stays whole on
        # every rank and is added after the all-reduce
        self.shared_split = init.tp > 1 and (f.shared_ffn // init.tp) % 64 == 0 and f.shared_ffn % init.tp == 0
        shared_init = init
        if init.tp > 1 and not self.shared_split:
            import copy
            shared_init = copy.copy(init)          # same seeded stream, no sharding
            shared_init.tp, shared_init.rank = 1, 0
        self.shared = (MlpLayer(t, shared_init, name + ".shared", width=f.shared_ffn, act=t.moe_act)
                       if t.shared_ffn else None)
        self.fc1_latent = init.linear(t.latent, t.hidden, "bf16", name + ".fc1_latent") if t.latent else None
        self.fc2_latent = init.linear(t.hidden, t.latent, "bf16", name + ".fc2_latent") if t.latent else None
        self.ep_size = ep_size
        self.tp = init.tp
        self.partial = False          # the expert-parallel forms reduce inside the layer

    def linears(self):
        out = [self.router]
        if self.shared is not None:
            out += self.shared.linears()
        out += [l for l in (self.fc1_latent, self.fc2_latent) if l is not None]
        return out

    experts_w3 = None      # optional 3-bit decode copy of the routed experts (attach_w3)

    def attach_w3(self, fc1=None, fc2=None) -> int:
        """3-bit decode copy of this rank's routed experts (int3, groups of 64, dequantisation fused into the grouped
        GEMM): calls of up to `W3_MAX_ROWS` rows stream it instead of the served stacks. `fc1` / `fc2`: calibrated
        `Int3G64` stacks over all experts' rows (weights/calibrate_model.py); default: nearest rounding of the served
        weights. Returns the bytes the copy adds. Reference: hibana/kernels/w3_moe.py, flashnext_w3_experts.py."""
        ew = self.experts
        n1, n2 = ew.n1, ew.fc2_rows
        if n1 % 128 or n2 % 128 or ew.hidden % 64 or ew.inter % 64:
            return 0            # the 3-bit tiles cover 128 rows x 64 columns
        dev = ew.fc1.q.device if ew.fmt == "nvfp4" else ew.fc1.device
        if fc1 is None:
            self.experts_w3 = moe.ExpertWeights.create(ew.dense(1), ew.dense(2), ew.act, "w3").to(dev)
        else:
            self.experts_w3 = moe.ExpertWeights.from_int3(fc1, fc2, ew.experts, ew.act, n2, dev)
        return self.experts_w3.fc1.numel() + self.experts_w3.fc2.numel()

    def _ew(self, x):
        """The expert stacks a call of x's row count reads."""
        from .linear import W3_MAX_ROWS
        return self.experts_w3 if self.experts_w3 is not None and x.shape[0] <= W3_MAX_ROWS else self.experts

    def _route(self, logits: torch.Tensor):
        """Top-k routing; with `expert_budget` set, decode-sized calls share experts across their rows."""
        t = self.t
        ids, w = moe.route(logits, t.top_k, sigmoid=t.router == "sigmoid", sel_bias=self.sel_bias, renorm=True,
                           scale=t.router_scale)
        cfg = cfgmod.current()
        if cfg.expert_budget > 0 and logits.shape[0] * t.top_k <= 16384 and logits.shape[0] <= 256:
            ids, w = moe.share_experts(ids, w, t.experts, min(cfg.expert_keep, t.top_k), cfg.expert_budget,
                                       scale=t.router_scale)
        return ids, w

    def forward(self, x, ctx=None, kv=None, states=None) -> torch.Tensor:
        t = self.t
        if overlap_ok(x, ctx):
            # decode-sized on one GPU: the latent projection and the shared expert do not depend on the routing, so
            # they run on a side stream beside router -> route -> plan -> grouped GEMMs (utils/streams.py)
            with streams.Branch(x) as br:
                lat = self.fc1_latent(x) if t.latent else None
                lat_ready = br.mark()
                shared = self.shared.forward(x) if self.shared is not None else None
            logits = gemm.linear_bf16(x, self.router.weight, epilogue=gemm.EPI_STORE_F32)
            ids, w = self._route(logits)
            if t.latent:
                br.wait(lat_ready, lat)
                y = moe.experts_forward(lat, ids, w, self._ew(lat), id_base=self.e_lo)
                out = self.fc2_latent(y)
                br.join(shared)
                return basic.add(out, shared) if shared is not None else out
            br.join(shared)
            return moe.experts_forward(x, ids, w, self._ew(x), shared=shared, id_base=self.e_lo)
        logits = gemm.linear_bf16(x, self.router.weight, epilogue=gemm.EPI_STORE_F32)
        ids, w = self._route(logits)
        shared = self.shared.forward(x) if self.shared is not None else None
        if shared is not None and self.shared_split and ctx is not None and ctx.comm is not None:
            shared = ctx.comm.all_reduce(shared)      # column / row split shared expert beside replicated experts
        if t.latent:
            lat = self.fc1_latent(x)
            y = moe.experts_forward(lat, ids, w, self._ew(lat), id_base=self.e_lo)
            out = self.fc2_latent(y)
            return basic.add(out, shared) if shared is not None else out
        return moe.experts_forward(x, ids, w, self._ew(x), shared=shared, id_base=self.e_lo)


def _moe_forward_ep(self, x, comm) -> torch.Tensor:
    """Replicated-activation expert parallelism: every rank runs its expert range on all tokens, the partial sums
    are all-reduced, and the (replicated) shared expert is added once afterwards."""
    t = self.t
    # the shared expert and the latent projection are plain local launches that do not depend on the routing: at
    # decode sizes they run on a side stream beside router -> route -> grouped GEMMs (the communicator's kernels stay
    # on the main stream)
    with streams.Branch(x, enabled=overlap_ok(x, None, comm_free=True)) as br:
        inp = self.fc1_latent(x) if t.latent else x
        lat_ready = br.mark()
        shared = self.shared.forward(x) if self.shared is not None else None
    logits = gemm.linear_bf16(x, self.router.weight, epilogue=gemm.EPI_STORE_F32)
    ids, w = self._route(logits)
    br.wait(lat_ready, inp if t.latent else None)
    part = moe.experts_forward(inp, ids, w, self._ew(inp), id_base=self.e_lo)
    if getattr(self, "tp", 1) > 1:
        # tensor parallel: the shared expert is column / row split too, so its partial sum joins the routed
        # experts' before the layer's one all-reduce; the latent up-projection is linear and moves in front of it
        if t.latent:
            part = self.fc2_latent(part)
        br.join(shared)
        if shared is not None and self.shared_split:
            part = basic.add(part, shared)
        out = comm.all_reduce(part)
        if shared is not None and not self.shared_split:
            out = basic.add(out, shared)                        # whole on every rank: added once, after the sum
        return out
    part = comm.all_reduce(part)
    out = self.fc2_latent(part) if t.latent else part
    br.join(shared)
    if shared is not None:
        out = basic.add(out, shared)
    return out


def _moe_forward_a2a(self, x, ep) -> torch.Tensor:
    """All-to-all expert parallelism (parallel/ep.py): `x` holds THIS rank's tokens only (attention ran data- or
    sequence-parallel); rows travel to the owners of their experts and the results come back. Every rank must
    call it, with an empty batch when it has no tokens."""
    t = self.t
    assert self.ep_size == ep.world and self.e_lo == ep.rank * ep.e_per, "the layer holds another expert range"
    # the shared expert (and the latent projection) are local launches: at decode sizes they run on a side stream
    # while the main stream routes and exchanges rows with the other ranks
    with streams.Branch(x, enabled=overlap_ok(x, None, comm_free=True)) as br:
        lat = self.fc1_latent(x) if t.latent else None
        lat_ready = br.mark()
        shared = self.shared.forward(x) if self.shared is not None and x.shape[0] else None
    logits = gemm.linear_bf16(x, self.router.weight, epilogue=gemm.EPI_STORE_F32)
    ids, w = self._route(logits)
    if t.latent:
        br.wait(lat_ready, lat)
        y = ep.forward(lat, ids, w, self.experts)
        out = self.fc2_latent(y)
        br.join(shared)
        return basic.add(out, shared) if shared is not None else out
    br.join(shared)
    return ep.forward(x, ids, w, self.experts, shared=shared)


MoeLayer.forward_ep = _moe_forward_ep
MoeLayer.forward_a2a = _moe_forward_a2a


def build_mixer(kind: str, t: Target, init: Init, counters: dict, name: str):
    if kind in (ATTN, GATED_ATTN):
        i = counters["kv"]
        counters["kv"] += 1
        return AttentionLayer(t, init, i, kind == GATED_ATTN, name)
    if kind in (MAMBA2, GDN):
        i = counters["state"]
        counters["state"] += 1
        return MambaLayer(t, init, i, name) if kind == MAMBA2 else GdnLayer(t, init, i, name)
    return None


def build_ffn(kind: str, t: Target, init: Init, name: str, ep_rank: int = 0, ep_size: int = 1):
    if kind == MLP:
        return MlpLayer(t, init, name)
    if kind in (MOE, LATENT_MOE):
        if t.weight_format == "ggml":
            from .bolt import BoltMoeLayer
            return BoltMoeLayer(t, init, name, ep_rank, ep_size)
        return MoeLayer(t, init, name, ep_rank, ep_size)
    return None
