"""Mixture-of-experts forward: route -> plan -> (gather | quantise) -> grouped fc1 (+act) -> grouped fc2 -> combine.

`ExpertWeights` holds all experts of a layer stacked: fc1 [E, 2I, H] with gate/up rows interleaved pairwise
(SwiGLU) or [E, I, H] (ReLU^2), fc2 [E, H, I]; bf16 or NVFP4 (one per-tensor scale per expert). The grouped GEMMs
are the grouped mode of the tcgen05 GEMM. With expert parallelism a rank plans only its own expert range
[e_lo, e_lo + e_n) and produces a partial sum (replicated-activation EP; the all-to-all variant lives in
parallel/ep.py). Reference: hibana/model/flashnext/moe.py:68-192, hibana/model/nemotron/moe.py:349-566,
hibana/kernels/w3_moe.py:194 (reference), hibana/kernels/csrc/w3_gemm.cu:640-1300.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as nv
from . import gemm, nvfp4

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_moe_route", [P, L, P, I, I, I, I, I, Fl, P, P, P])
nv.register("hb_quant_nvfp4_pairs", [P, L, P, I, I, I, I, P, P, P, P])
nv.register("hb_moe_plan", [P, I, I, I, I, I, I, P, P, P, P, I, P, I, P, P, I, P])
nv.register("hb_moe_gather", [P, L, P, P, P, I, I, P])
nv.register("hb_moe_combine", [P, L, P, P, P, L, P, L, I, I, I, P])
nv.register("hb_gemm_grouped", [I, P, P, P, P, I, I, I, I, P, L, P, I, P, P, I, P, I, I, I, P, P, I, P])
nv.register("hb_quant_nvfp4_rows", [P, L, I, I, I, P, P, P, I, P, P, P])


def route_ref(logits: torch.Tensor, topk: int, *, sigmoid: bool = False, sel_bias: Optional[torch.Tensor] = None,
              renorm: bool = True, scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    lg = logits.float()
    if sigmoid:
        score = torch.sigmoid(lg)
        sel = score + (sel_bias.float() if sel_bias is not None else 0.0)
    else:
        score = torch.softmax(lg, dim=-1)
        sel = score
    # stable descending order = lowest index wins ties, like the kernel
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :topk]
    w = score.gather(1, order)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return order.int(), (w * scale).float()


def route(logits: torch.Tensor, topk: int, *, sigmoid: bool = False, sel_bias: Optional[torch.Tensor] = None,
          renorm: bool = True, scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 logits [T, E] -> (ids int32 [T, k], weights fp32 [T, k])."""
    t, e = logits.shape
    if nv.use_native(logits):
        ids = torch.empty(t, topk, dtype=torch.int32, device=logits.device)
        w = torch.empty(t, topk, dtype=torch.float32, device=logits.device)
        nv.check(nv.lib().hb_moe_route(logits.data_ptr(), logits.stride(0), nv.ptr(sel_bias), t, e, topk,
                                       int(sigmoid), int(renorm), scale, ids.data_ptr(), w.data_ptr(), nv.stream()),
                 "hb_moe_route")
        return ids, w
    return route_ref(logits, topk, sigmoid=sigmoid, sel_bias=sel_bias, renorm=renorm, scale=scale)


nv.register("hb_moe_share", [P, P, I, I, I, I, I, nv.F, P])


def share_experts_ref(ids: torch.Tensor, weights: torch.Tensor, experts: int, keep: int, budget: int,
                      scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Plain PyTorch `share_experts` (same integer score sums, same tie rule)."""
    rows, k = ids.shape
    ids, weights = ids.clone().cpu(), weights.clone().cpu().float()
    score = torch.zeros(experts, dtype=torch.int64)
    core = torch.zeros(experts, dtype=torch.bool)
    for r in range(rows):
        tot = torch.zeros((), dtype=torch.float32)
        for q in range(k):
            tot = tot + weights[r, q]
        for j in range(k):
            e = int(ids[r, j])
            if 0 <= e < experts:
                w = weights[r, j] / tot if float(tot) > 0 else torch.zeros(())
                score[e] += int((w * torch.tensor(16777216.0)).to(torch.int64))
                if j < keep:
                    core[e] = True
    need = budget - int(core.sum())
    chosen = core.clone()
    if need > 0:
        rest = [(-int(score[e]), e) for e in range(experts) if not core[e] and int(score[e]) > 0]
        for _, e in sorted(rest)[:need]:
            chosen[e] = True
    for r in range(rows):
        first = int(ids[r, 0])
        kept = [(int(ids[r, j]), weights[r, j].clone()) for j in range(k)
                if 0 <= int(ids[r, j]) < experts and chosen[int(ids[r, j])]]
        tot = torch.zeros((), dtype=torch.float32)
        for _, w in kept:
            tot = tot + w
        inv = torch.tensor(scale, dtype=torch.float32) / tot if float(tot) > 0 else torch.zeros(())
        for j in range(k):
            if j < len(kept):
                ids[r, j], weights[r, j] = kept[j][0], kept[j][1] * inv
            else:
                ids[r, j], weights[r, j] = first, 0.0
    return ids, weights


def share_experts(ids: torch.Tensor, weights: torch.Tensor, experts: int, keep: int, budget: int,
                  scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Budgeted expert sharing for decode-sized batches: the call as a whole uses at most `budget` distinct experts
    (more only when the rows' guaranteed best `keep` choices alone exceed it). Every row keeps its best `keep`;
    the remaining budget goes to the experts with the largest routing weight summed over the call; a row then uses
    those of its top-k inside the set, weights renormalised over them (times `scale`), and repeats its best expert
    at weight 0 in the slots it lost. Lossy by design (fewer experts' weights are streamed per step); rows that
    keep all their choices keep their weights up to the renormalisation. ids int32 / weights fp32 [rows, k] from
    `route`; returns new tensors. Reference: hibana/model/nemotron/moe.py:171-306 (`route_budget`),
    hibana/kernels/flashnext_fused.py:412-506."""
    rows, k = ids.shape
    if nv.use_native(ids) and experts <= 1024 and rows * k <= 16384:
        ids, weights = ids.clone(), weights.clone()
        nv.check(nv.lib().hb_moe_share(ids.data_ptr(), weights.data_ptr(), rows, k, experts, keep, budget, scale,
                                       nv.stream()), "hb_moe_share")
        return ids, weights
    i2, w2 = share_experts_ref(ids, weights, experts, keep, budget, scale)
    return i2.to(ids.device), w2.to(weights.device)


@dataclass
class ExpertWeights:
    """Stacked expert matrices. fc1: [E * n1, H] rows (n1 = 2I interleaved for SwiGLU, I for ReLU^2); fc2:
    [E * H_out, I]. For NVFP4 `*_q` are Nvfp4Tensors over the stacked rows and `*_alpha` [E] = act_scale * w_scale."""
    experts: int
    hidden: int           # input width of fc1 / output width of fc2
    inter: int
    act: str              # swiglu | relu2
    fmt: str              # bf16 | nvfp4
    fc1: object
    fc2: object
    fc1_alpha: Optional[torch.Tensor] = None
    fc2_alpha: Optional[torch.Tensor] = None
    fc1_in_scale: Optional[torch.Tensor] = None
    fc2_in_scale: Optional[torch.Tensor] = None

    @property
    def n1(self) -> int:
        return 2 * self.inter if self.act == "swiglu" else self.inter

    @classmethod
    def create(cls, fc1: torch.Tensor, fc2: torch.Tensor, act: str, fmt: str, in_amax: float = 8.0,
               mid_amax: float = 8.0) -> "ExpertWeights":
        """fc1 [E, n1, H], fc2 [E, H, I] (fp32 / bf16)."""
        e, n1, h = fc1.shape
        inter = fc2.shape[2]
        if fmt == "bf16":
            return cls(e, h, inter, act, fmt, fc1.reshape(e * n1, h).to(torch.bfloat16).contiguous(),
                       fc2.reshape(e * fc2.shape[1], inter).to(torch.bfloat16).contiguous())
        dev = fc1.device
        if fmt == "w3":
            # 3-bit experts (groups of 64, scale + zero): one tile stack over all experts' rows; an expert's rows
            # are a multiple of 128, so expert boundaries fall on tile boundaries
            from ..weights.w3 import Int3G64
            assert n1 % 128 == 0 and fc2.shape[1] % 128 == 0
            # quantised where the weights are (a full-size layer's stacks never visit the host)
            q1 = Int3G64.quantize(fc1.reshape(e * n1, h))
            q2 = Int3G64.quantize(fc2.reshape(e * fc2.shape[1], inter))
            return cls.from_int3(q1, q2, e, act, fc2.shape[1], dev)

        def quant(w):   # per-expert scale, stacked rows
            parts = [nvfp4.quantize_weight(w[i]) for i in range(w.shape[0])]
            q = torch.cat([p.q for p in parts], 0)
            sfb = torch.cat([nvfp4.unswizzle_sf(p.sf, p.rows, p.k // 16) for p in parts], 0)
            gs = torch.stack([p.gscale.reshape(()) for p in parts]).float()
            return nvfp4.Nvfp4Tensor(q, nvfp4.swizzle_sf(sfb), gs, q.shape[0], w.shape[2]), gs

        q1, g1 = quant(fc1)
        q2, g2 = quant(fc2)
        s1 = torch.tensor([in_amax / (6 * 448.0)], dtype=torch.float32, device=dev)
        s2 = torch.tensor([mid_amax / (6 * 448.0)], dtype=torch.float32, device=dev)
        return cls(e, h, inter, act, fmt, q1, q2, (g1 * s1).contiguous(), (g2 * s2).contiguous(), s1, s2)

    @classmethod
    def from_int3(cls, q1, q2, experts: int, act: str, fc2_rows: int, device) -> "ExpertWeights":
        """3-bit expert stacks from two `Int3G64` matrices over all experts' rows (fc1 [E * n1, H], fc2
        [E * fc2_rows, I]): nearest-rounded (`create`) or calibrated (weights/calibrate_model.py)."""
        h, inter = q1.shape[1], q2.shape[1]
        out = cls(experts, h, inter, act, "w3", q1.tiles().to(device), q2.tiles().to(device))
        out.w3 = (q1, q2)
        out.fc2_rows_ = fc2_rows
        return out

    def dense(self, which: int) -> torch.Tensor:
        """Dequantised stacked matrix [E, n, k] (fp32) for the reference path."""
        w = self.fc1 if which == 1 else self.fc2
        n = self.n1 if which == 1 else self.fc2_rows
        if self.fmt == "w3":
            return self.w3[which - 1].dequantize().view(self.experts, n, -1).to(w.device)
        if self.fmt == "bf16":
            return w.float().view(self.experts, n, -1)
        sfb = nvfp4.unswizzle_sf(w.sf, w.rows, w.k // 16)
        out = torch.empty(w.rows, w.k, dtype=torch.float32, device=w.q.device)
        for e in range(self.experts):
            sl = slice(e * n, (e + 1) * n)
            out[sl] = nvfp4.dequantize_ref(w.q[sl], sfb[sl], w.gscale[e])
        return out.view(self.experts, n, -1)

    @property
    def fc2_rows(self) -> int:
        if self.fmt == "w3":
            return self.fc2_rows_
        return (self.fc2.shape[0] if self.fmt == "bf16" else self.fc2.rows) // self.experts

    def slice(self, e_lo: int, e_n: int) -> "ExpertWeights":
        """The experts [e_lo, e_lo + e_n) as views (what one expert-parallel rank keeps)."""
        n1, n2 = self.n1, self.fc2_rows

        def rows(w, n):
            if self.fmt == "bf16":
                return w[e_lo * n:(e_lo + e_n) * n]
            assert n % 128 == 0, "scale blocks cover 128 rows: expert boundaries must fall on them"
            return nvfp4.Nvfp4Tensor(w.q[e_lo * n:(e_lo + e_n) * n], w.sf[e_lo * n // 128:(e_lo + e_n) * n // 128],
                                     w.gscale[e_lo:e_lo + e_n], e_n * n, w.k)

        cut = (lambda v: v[e_lo:e_lo + e_n].contiguous()) if self.fmt != "bf16" else (lambda v: v)
        return ExpertWeights(e_n, self.hidden, self.inter, self.act, self.fmt, rows(self.fc1, n1), rows(self.fc2, n2),
                             cut(self.fc1_alpha), cut(self.fc2_alpha), self.fc1_in_scale, self.fc2_in_scale)

    def to(self, device) -> "ExpertWeights":
        def mv(x):
            if isinstance(x, nvfp4.Nvfp4Tensor):
                return nvfp4.Nvfp4Tensor(x.q.to(device), x.sf.to(device), x.gscale.to(device), x.rows, x.k)
            return x.to(device) if isinstance(x, torch.Tensor) else x
        out = ExpertWeights(self.experts, self.hidden, self.inter, self.act, self.fmt, mv(self.fc1), mv(self.fc2),
                            mv(self.fc1_alpha), mv(self.fc2_alpha), mv(self.fc1_in_scale), mv(self.fc2_in_scale))
        if self.fmt == "w3":
            out.w3, out.fc2_rows_ = self.w3, self.fc2_rows_
        return out


def _act(h1: torch.Tensor, act: str) -> torch.Tensor:
    if act == "swiglu":
        return F.silu(h1[..., 0::2]) * h1[..., 1::2]
    return torch.relu(h1) ** 2


def experts_ref(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: ExpertWeights,
                shared: Optional[torch.Tensor] = None, e_lo: int = 0, e_n: Optional[int] = None,
                id_base: int = 0) -> torch.Tensor:
    """Plain PyTorch: per (token, k) pair run the selected expert; sum in selection order."""
    e_n = ew.experts if e_n is None else e_n
    t = x.shape[0]
    w1, w2 = ew.dense(1), ew.dense(2)
    xf = x.float()
    if ew.fmt == "nvfp4":   # same activation quantisation as the kernel path
        q, sfb = nvfp4.quantize_ref(x, ew.fc1_in_scale)
        xf = nvfp4.dequantize_ref(q, sfb, ew.fc1_in_scale)
    out = torch.zeros(t, ew.fc2_rows, dtype=torch.float32, device=x.device)
    for ti in range(t):
        for k in range(ids.shape[1]):
            e = int(ids[ti, k]) - id_base
            if e < e_lo or e >= e_lo + e_n:
                continue
            h1 = (xf[ti] @ w1[e].t()).to(torch.bfloat16).float() if ew.act != "swiglu" else xf[ti] @ w1[e].t()
            mid = _act(h1, ew.act).to(torch.bfloat16)
            if ew.fmt == "nvfp4":
                q, sfb = nvfp4.quantize_ref(mid.view(1, -1), ew.fc2_in_scale)
                midf = nvfp4.dequantize_ref(q, sfb, ew.fc2_in_scale)[0]
            else:
                midf = mid.float()
            y = (midf @ w2[e].t()).to(torch.bfloat16).float()
            out[ti] += float(weights[ti, k]) * y
    if shared is not None:
        out += shared.float()
    return out.to(torch.bfloat16)


def tile_hint(pairs: int, experts: int, max_rows: int, fmt: str) -> int:
    """Token-tile width for the grouped GEMMs from the EXPECTED rows per expert (the grid still covers the worst
    case; chunks beyond an expert's rows exit at once). Block-scaled FP4 needs whole 128-row scale blocks per chunk
    unless the expert fits one chunk."""
    avg = max(1, -(-pairs // max(experts, 1)))
    bn = 16
    while bn < min(avg + avg // 4, 128):     # 128 at most: up to that width two CTAs share an SM (csrc/gemm.cu Cfg)
        bn *= 2
    if fmt == "nvfp4" and bn < 128 and max_rows > bn:
        bn = 128
    return bn


def experts_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: ExpertWeights, *,
                    shared: Optional[torch.Tensor] = None, e_lo: int = 0, e_n: Optional[int] = None,
                    id_base: int = 0) -> torch.Tensor:
    """x [T, H] bf16, ids / weights [T, k] -> [T, H_out] bf16 (sum of the routed experts (+ shared)). `ew` holds
    the experts `id_base` .. `id_base + ew.experts - 1` of the numbering `ids` use (an expert-parallel rank keeps a
    range); of those, only [e_lo, e_lo + e_n) run. Pairs routed elsewhere add nothing."""
    e_n = ew.experts if e_n is None else e_n
    if not nv.use_native(x):
        return experts_ref(x, ids, weights, ew, shared, e_lo, e_n, id_base)
    lib = nv.lib()
    t, h = x.shape
    topk = ids.shape[1]
    dev = x.device
    e = ew.experts
    rows_cap = ((t * topk + 127) // 128) * 128 + min(e_n, t * topk) * 128
    max_rows = min(t, 1 << 30)                  # an expert can receive every token once
    bn_hint = tile_hint(t * topk, e_n, max_rows, ew.fmt)
    bn_full = 16
    while bn_full < max_rows and bn_full < 256:
        bn_full *= 2
    bn_hint = min(bn_hint, bn_full)            # the tile width the grouped GEMMs will use
    # compact (expert, chunk) work list: the GEMM grids cover the tiles that have rows, not experts x worst case
    tile_cap = -(-(t * topk) // bn_hint) + min(e_n, t * topk)
    tiles = torch.empty(tile_cap, dtype=torch.int32, device=dev)
    n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    tl = (tiles.data_ptr(), n_tiles.data_ptr(), tile_cap)
    cnt = torch.empty(e, dtype=torch.int32, device=dev)
    start = torch.empty(e, dtype=torch.int32, device=dev)
    pos = torch.empty(t * topk, dtype=torch.int32, device=dev)
    src = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    st = nv.device_state(dev).status
    nv.check(lib.hb_moe_plan(ids.data_ptr(), t, topk, e, e_lo, e_n, id_base, cnt.data_ptr(), start.data_ptr(), pos.data_ptr(),
                             src.data_ptr(), rows_cap, total.data_ptr(), bn_hint, tiles.data_ptr(),
                             n_tiles.data_ptr(), tile_cap, nv.stream()), "hb_moe_plan")
    n1, h_out = ew.n1, ew.fc2_rows
    epi1 = gemm.EPI_SILU_MUL if ew.act == "swiglu" else gemm.EPI_RELU2 if ew.act == "relu2" else gemm.EPI_STORE
    mid_cols = ew.inter
    h1 = torch.empty(rows_cap, mid_cols if ew.act == "swiglu" else n1, dtype=torch.bfloat16, device=dev)
    y = torch.empty(rows_cap, h_out, dtype=torch.bfloat16, device=dev)
    if ew.fmt in ("bf16", "w3"):
        kind = 0 if ew.fmt == "bf16" else 3      # 3: dequant-fused 3-bit experts (csrc/gemm.cu kind w3, grouped)
        xs = torch.empty(rows_cap, h, dtype=torch.bfloat16, device=dev)
        nv.check(lib.hb_moe_gather(x.data_ptr(), x.stride(0), src.data_ptr(), total.data_ptr(), xs.data_ptr(),
                                   rows_cap, h, nv.stream()), "hb_moe_gather")
        nv.check(lib.hb_gemm_grouped(kind, ew.fc1.data_ptr(), xs.data_ptr(), None, None, e, n1, rows_cap, h,
                                     h1.data_ptr(), h1.stride(0), None, epi1, start.data_ptr(), cnt.data_ptr(),
                                     max_rows, st.data_ptr(), 0, 0, bn_hint, *tl, nv.stream()), "hb_gemm_grouped")
        mid = h1                                # the activation (SwiGLU or squared ReLU) ran in the GEMM epilogue
        nv.check(lib.hb_gemm_grouped(kind, ew.fc2.data_ptr(), mid.data_ptr(), None, None, e, h_out, rows_cap,
                                     ew.inter, y.data_ptr(), y.stride(0), None, gemm.EPI_STORE, start.data_ptr(),
                                     cnt.data_ptr(), max_rows, st.data_ptr(), 0, 0, bn_hint, *tl, nv.stream()), "hb_gemm_grouped")
    else:
        q1, sf1 = nvfp4._alloc(rows_cap, h, dev)
        # few pairs (decode, verify): quantise by pair, not by row of the padded buffer (most of which is padding
        # of the 128-row expert segments that the GEMM never stores from)
        by_pair = t * topk * 8 <= rows_cap
        if by_pair:
            nv.check(lib.hb_quant_nvfp4_pairs(x.data_ptr(), x.stride(0), pos.data_ptr(), t * topk, topk, h,
                                              sf1.shape[1], ew.fc1_in_scale.data_ptr(), q1.data_ptr(),
                                              sf1.data_ptr(), nv.stream()), "hb_quant_nvfp4_pairs")
        else:
            nv.check(lib.hb_quant_nvfp4_rows(x.data_ptr(), x.stride(0), rows_cap, h, sf1.shape[1],
                                             ew.fc1_in_scale.data_ptr(), q1.data_ptr(), sf1.data_ptr(), 0,
                                             src.data_ptr(), total.data_ptr(), nv.stream()), "hb_quant_nvfp4_rows")
        nv.check(lib.hb_gemm_grouped(1, ew.fc1.q.data_ptr(), q1.data_ptr(), ew.fc1.sf.data_ptr(), sf1.data_ptr(), e,
                                     n1, rows_cap, h, h1.data_ptr(), h1.stride(0), ew.fc1_alpha.data_ptr(), epi1,
                                     start.data_ptr(), cnt.data_ptr(), max_rows, st.data_ptr(), ew.fc1.ka,
                                     sf1.shape[1], bn_hint, *tl, nv.stream()), "hb_gemm_grouped")
        mid = h1                                # the activation (SwiGLU or squared ReLU) ran in the GEMM epilogue
        q2, sf2 = nvfp4._alloc(rows_cap, ew.inter, dev)
        if by_pair:
            nv.check(lib.hb_quant_nvfp4_pairs(mid.data_ptr(), mid.stride(0), pos.data_ptr(), t * topk, 0, ew.inter,
                                              sf2.shape[1], ew.fc2_in_scale.data_ptr(), q2.data_ptr(),
                                              sf2.data_ptr(), nv.stream()), "hb_quant_nvfp4_pairs")
        else:
            nv.check(lib.hb_quant_nvfp4_rows(mid.data_ptr(), mid.stride(0), rows_cap, ew.inter, sf2.shape[1],
                                             ew.fc2_in_scale.data_ptr(), q2.data_ptr(), sf2.data_ptr(), 0, None,
                                             total.data_ptr(), nv.stream()), "hb_quant_nvfp4_rows")
        nv.check(lib.hb_gemm_grouped(1, ew.fc2.q.data_ptr(), q2.data_ptr(), ew.fc2.sf.data_ptr(), sf2.data_ptr(), e,
                                     h_out, rows_cap, ew.inter, y.data_ptr(), y.stride(0), ew.fc2_alpha.data_ptr(),
                                     gemm.EPI_STORE, start.data_ptr(), cnt.data_ptr(), max_rows, st.data_ptr(),
                                     ew.fc2.ka, sf2.shape[1], bn_hint, *tl, nv.stream()), "hb_gemm_grouped")
    out = torch.empty(t, h_out, dtype=torch.bfloat16, device=dev)
    nv.check(lib.hb_moe_combine(y.data_ptr(), y.stride(0), pos.data_ptr(), weights.data_ptr(), nv.ptr(shared),
                                shared.stride(0) if shared is not None else 0, out.data_ptr(), out.stride(0), t, topk,
                                h_out, nv.stream()), "hb_moe_combine")
    return out
