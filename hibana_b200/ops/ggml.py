"""Linear layers over GGML block formats kept in their checkpoint bytes (csrc/ggml.cu).

`PackedLinear` holds a [N, K] matrix as Q8_0, IQ2_XXS or IQ2_XS blocks on the device. Products with up to 8
activation rows (decode, short verify blocks) run the decode-fused kernel: every weight byte is read once and expanded
in registers, so a step moves 2.06 to 8.5 bits per weight. Larger products expand the matrix to bf16 (transient,
row-blocked) and run on the tcgen05 GEMM. `PackedExperts` is the stacked form of a mixture-of-experts layer: the
(token, expert) pairs of a decode step are one grouped launch per projection. The IQ2 lattice tables are part of the
file format and come with the checkpoint (`grids`); nothing here invents them.
Reference: hibana/model/bolt/linear.py:1-159 (PackedLinear), hibana/kernels/iq2_moe.py:34-240,
hibana/kernels/ggml_bf16.py:33-174.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import _native as nv
from ..weights import ggml as fmt
from . import gemm

P, I, L = nv.P, nv.I, nv.L
nv.register("hb_ggml_gemv", [I, P, L, I, I, P, L, I, P, I, P, L, P])
nv.register("hb_ggml_gemv_pairs", [I, P, L, L, I, I, P, L, P, P, P, I, I, P, L, P])
nv.register("hb_ggml_dequant", [I, P, L, I, I, I, P, P, P])

GEMV_ROWS = 8
TYPES = {"q8_0": fmt.T_Q8_0, "iq2_xxs": fmt.T_IQ2_XXS, "iq2_xs": fmt.T_IQ2_XS}


def row_bytes(gtype: int, k: int) -> int:
    per, nbytes = fmt.BLOCK[gtype]
    if k % per:
        raise ValueError(f"{fmt.NAMES[gtype]} rows hold whole blocks of {per} weights, K = {k} does not")
    return k // per * nbytes


class PackedLinear:
    def __init__(self, raw: torch.Tensor, gtype: int | str, n: int, k: int, grid: Optional[torch.Tensor] = None,
                 name: str = ""):
        """raw: uint8 [N * row_bytes] (or [N, row_bytes]) block bytes; grid: the format's lattice table uint8
        [256 or 512, 8] for the IQ2 types."""
        self.gtype = TYPES[gtype] if isinstance(gtype, str) else int(gtype)
        self.n, self.k, self.name = n, k, name
        self.row_bytes = row_bytes(self.gtype, k)
        self.raw = raw.reshape(n, self.row_bytes).contiguous()
        if self.gtype != fmt.T_Q8_0:
            want = 256 if self.gtype == fmt.T_IQ2_XXS else 512
            if grid is None or tuple(grid.shape) != (want, 8):
                raise ValueError(f"{fmt.NAMES[self.gtype]} needs its lattice table: uint8 [{want}, 8]")
            grid = grid.to(self.raw.device, torch.uint8).contiguous()
        self.grid = grid
        self.out_features, self.in_features, self.fmt = n, k, fmt.NAMES[self.gtype]

    def nbytes(self) -> int:
        return self.raw.numel()

    def to(self, device) -> "PackedLinear":
        self.raw = self.raw.to(device)
        self.grid = self.grid.to(device) if self.grid is not None else None
        return self

    def shard(self, rows=None, cols: Optional[slice] = None) -> "PackedLinear":
        """A tensor-parallel shard as block bytes of this matrix, nothing requantised: `rows` (slice or index
        tensor) keeps output features, `cols` (a contiguous slice of whole blocks) keeps input features."""
        raw = self.raw
        if rows is not None:
            raw = raw[rows.to(raw.device) if isinstance(rows, torch.Tensor) else rows]
        k = self.k
        if cols is not None:
            per, nbytes = fmt.BLOCK[self.gtype]
            c0, c1, step = cols.indices(self.k)
            if step != 1 or c0 % per or c1 % per:
                raise ValueError(f"{self.fmt}: a column shard must be whole blocks of {per} weights, got [{c0}, {c1})")
            raw, k = raw[:, c0 // per * nbytes:c1 // per * nbytes], c1 - c0
        raw = raw.contiguous()
        return type(self)(raw, self.gtype, raw.shape[0], k, self.grid, name=self.name)

    def dequantize(self, row0: int = 0, rows: Optional[int] = None) -> torch.Tensor:
        """bf16 [rows, K] of rows [row0, row0 + rows)."""
        rows = self.n - row0 if rows is None else rows
        if nv.use_native(self.raw):
            out = torch.empty(rows, self.k, dtype=torch.bfloat16, device=self.raw.device)
            nv.check(nv.lib().hb_ggml_dequant(self.gtype, self.raw.data_ptr(), self.row_bytes, row0, rows, self.k,
                                              nv.ptr(self.grid), out.data_ptr(), nv.stream()), "hb_ggml_dequant")
            return out
        grids = {fmt.NAMES[self.gtype]: self.grid.cpu().numpy()} if self.grid is not None else None
        w = fmt.dequantize(self.raw[row0:row0 + rows].cpu().numpy().reshape(-1), self.gtype, (rows, self.k), grids)
        return torch.from_numpy(w).to(torch.bfloat16).to(self.raw.device)

    def __call__(self, x: torch.Tensor, relu2: bool = False) -> torch.Tensor:
        m = x.shape[0]
        if nv.use_native(x) and m <= GEMV_ROWS and x.stride(0) % 8 == 0:
            mp = 1 if m == 1 else 2 if m == 2 else 4 if m <= 4 else 8
            xp = x if mp == m else torch.cat((x, x.new_zeros(mp - m, x.shape[1])), 0)
            y = torch.empty(mp, self.n, dtype=torch.bfloat16, device=x.device)
            nv.check(nv.lib().hb_ggml_gemv(self.gtype, self.raw.data_ptr(), self.row_bytes, self.n, self.k,
                                           xp.data_ptr(), xp.stride(0), mp, nv.ptr(self.grid), int(relu2),
                                           y.data_ptr(), y.stride(0), nv.stream()), "hb_ggml_gemv")
            return y[:m]
        # prefill-sized: expand 4096 weight rows at a time and run the tensor-core GEMM on each block
        outs = []
        for r0 in range(0, self.n, 4096):
            wb = self.dequantize(r0, min(4096, self.n - r0))
            outs.append(gemm.linear_bf16(x, wb) if x.is_cuda else (x.float() @ wb.float().t()).to(torch.bfloat16))
        y = outs[0] if len(outs) == 1 else torch.cat(outs, 1)
        return (torch.relu(y.float()) ** 2).to(torch.bfloat16) if relu2 else y


class PackedExperts:
    """E stacked expert matrices per projection (fc1 [E, I, H] with squared ReLU, fc2 [E, H, I]) in GGML blocks."""

    def __init__(self, fc1: PackedLinear, fc2: PackedLinear, experts: int):
        assert fc1.n % experts == 0 and fc2.n % experts == 0
        self.fc1, self.fc2, self.experts = fc1, fc2, experts
        self.inter, self.hidden = fc1.n // experts, fc2.n // experts
        self.total = experts          # experts of the whole layer (more than `experts` on a rank that holds a range)

    def slice(self, e_lo: int, e_n: int) -> "PackedExperts":
        """The experts [e_lo, e_lo + e_n): what one rank keeps when the experts are split by range."""
        part = PackedExperts(self.fc1.shard(rows=slice(e_lo * self.inter, (e_lo + e_n) * self.inter)),
                             self.fc2.shard(rows=slice(e_lo * self.hidden, (e_lo + e_n) * self.hidden)), e_n)
        part.total = self.total
        return part

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, id_base: int = 0) -> torch.Tensor:
        """x [T, H] bf16, ids int32 [T, k], weights fp32 [T, k] -> [T, H] bf16: sum_k w * fc2_e(relu(fc1_e x)^2).
        `id_base`: global id of this object's first expert; pairs routed to experts it does not hold add nothing
        (the result is then this rank's partial sum)."""
        t, k = ids.shape
        pairs = t * k
        gids, gweights = ids, weights
        if id_base or self.total > self.experts:
            local = ids - id_base
            mine = (local >= 0) & (local < self.experts)
            ids = torch.where(mine, local, torch.full_like(local, -1))
            weights = torch.where(mine, weights, torch.zeros_like(weights))
            sharded = True
        else:
            sharded = False
        if nv.use_native(x) and pairs <= 4096:
            dev = x.device
            pe = ids.reshape(-1).contiguous()
            pr = torch.arange(t, dtype=torch.int32, device=dev).repeat_interleave(k)
            own = torch.arange(pairs, dtype=torch.int32, device=dev)
            h1 = torch.empty(pairs, self.inter, dtype=torch.bfloat16, device=dev)
            # the kernel skips pairs with a negative expert: their rows must read zero in the weighted sum below
            y = (torch.zeros if sharded else torch.empty)(pairs, self.hidden, dtype=torch.bfloat16, device=dev)
            lib = nv.lib()
            for lin, src, rows, relu2, out, n in ((self.fc1, x, pr, 1, h1, self.inter), (self.fc2, h1, own, 0, y, self.hidden)):
                nv.check(lib.hb_ggml_gemv_pairs(lin.gtype, lin.raw.data_ptr(), lin.row_bytes, lin.row_bytes * n, n,
                                                lin.k, src.data_ptr(), src.stride(0), nv.ptr(lin.grid), pe.data_ptr(),
                                                rows.data_ptr(), pairs, relu2, out.data_ptr(), out.stride(0),
                                                nv.stream()), "hb_ggml_gemv_pairs")
            return (y.view(t, k, -1).float() * weights[:, :, None]).sum(1).to(torch.bfloat16)
        if nv.use_native(x):
            # prefill-sized: every expert has rows, so the two stacks are expanded to bf16 once (transient: a layer's
            # experts, a few GB) and the ranked plan + grouped tensor-core GEMMs of the NVFP4 families do the rest.
            # One kernel per stack reads every block once; nothing visits the host.
            from . import moe
            ew = moe.ExpertWeights(self.experts, self.fc1.k, self.inter, "relu2", "bf16",
                                   self.fc1.dequantize(0, self.fc1.n), self.fc2.dequantize(0, self.fc2.n))
            return moe.experts_forward(x, gids, gweights, ew, id_base=id_base)
        out = torch.zeros(t, self.hidden, dtype=torch.float32, device=x.device)
        for e in ids.unique().tolist():
            if e < 0:
                continue
            tok, slot = (ids == e).nonzero(as_tuple=True)
            w1 = self.fc1.dequantize(e * self.inter, self.inter).float()
            w2 = self.fc2.dequantize(e * self.hidden, self.hidden).float()
            h = (torch.relu(x[tok].float() @ w1.t()) ** 2).to(torch.bfloat16).float()
            yy = (h @ w2.t()).to(torch.bfloat16).float()
            out.index_add_(0, tok, yy * weights[tok, slot][:, None])
        return out.to(torch.bfloat16)


def random_blocks(gtype: int | str, n: int, k: int, seed: int = 0, scale: float = 0.02) -> torch.Tensor:
    """Valid random block bytes for an [N, K] matrix (synthetic weights: every byte pattern is a legal block; only
    the fp16 block scale is kept small and finite)."""
    gtype = TYPES[gtype] if isinstance(gtype, str) else int(gtype)
    rb = row_bytes(gtype, k)
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n, rb), dtype=np.uint8)
    per, nbytes = fmt.BLOCK[gtype]
    d = (rng.random((n, k // per), dtype=np.float32) * scale + scale * 0.1).astype(np.float16).view(np.uint8)
    blocks = raw.reshape(n, k // per, nbytes)
    blocks[:, :, :2] = d.reshape(n, k // per, 2)
    return torch.from_numpy(blocks.reshape(n, rb).copy())
