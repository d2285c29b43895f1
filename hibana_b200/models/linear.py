"""Linear layers over the quantised weight formats (bf16, NVFP4; w3 and FP8 plug in through the same interface).

A `Linear` owns one weight matrix [N, K] in its storage format plus the static activation scale NVFP4 needs.
`norm_linear` runs (residual add +) RMSNorm and the following projection with the norm fused into the
activation quantiser when the projection is NVFP4. The reference's equivalents are Fp8Linear / Nvfp4Linear
(hibana/weights/modelopt.py:108-184) called through hibana/kernels/ops.py:56-128.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .. import config as cfgmod
from ..ops import basic, gemm, gemv, nvfp4
from ..ops.nvfp4 import Nvfp4Tensor

Activation = Union[torch.Tensor, Nvfp4Tensor]
# The GEMV decodes weights in registers, which costs ~3 issue slots per weight: above a few tens of MB the tcgen05
# GEMM streams faster (4.8 vs 2.9 TB/s at 100 MB), below it the GEMM's fixed cost dominates (15 vs 10 us at 20 MB).
GEMV_MAX_WEIGHTS = 48 * 1024 * 1024
GEMV_MAX_ROWS = 4
W3_MAX_ROWS = 256        # token rows up to which the 3-bit copy is used (the dequant-fused kernel's tile limit)


def interleave_pairs(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up -> [2I, K] with rows g0, u0, g1, u1, ... (what the SiLU-mul GEMM epilogue expects)."""
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()


class Linear:
    """y = x @ W.T. `fmt` is 'bf16' or 'nvfp4'. `input_amax` is the calibrated activation range (NVFP4 only)."""

    def __init__(self, weight: torch.Tensor, fmt: str = "bf16", input_amax: float = 8.0, name: str = ""):
        self.fmt = fmt
        self.name = name
        self.out_features, self.in_features = weight.shape
        self.calibrating = False
        self.seen_amax = 0.0
        self.w3 = None              # optional 3-bit decode copy (ops/w3gemm.py W3Linear): rows <= W3_MAX_ROWS use it
        if fmt == "bf16":
            self.weight = weight.to(torch.bfloat16).contiguous()
            self.wq = None
        elif fmt == "nvfp4":
            self.wq = nvfp4.quantize_weight(weight)
            self.weight = None
            self.set_input_amax(input_amax)
        else:
            raise ValueError(f"unknown linear format {fmt!r}")

    @classmethod
    def sharded(cls, weight: torch.Tensor, fmt: str, rows: Optional[slice] = None, cols: Optional[slice] = None,
                name: str = "") -> "Linear":
        """A tensor-parallel shard that is bitwise a slice of the unsharded layer: the full matrix is quantised
        with its own per-tensor scale and then rows (output features) and / or columns (input features, on
        16-element block boundaries) are cut out. Reference: hibana/weights/sharding.py:15-19,
        hibana/model/flashnext/linear.py:31-43."""
        rows = slice(None) if rows is None else rows
        cols = slice(None) if cols is None else cols
        if fmt != "nvfp4":
            return cls(weight[rows][:, cols], fmt, name=name)
        full = nvfp4.quantize_weight(weight)
        sfb = nvfp4.unswizzle_sf(full.sf, full.rows, full.k // 16)
        c0 = cols.start or 0
        c1 = cols.stop if cols.stop is not None else full.k
        assert c0 % 16 == 0 and c1 % 16 == 0
        q = full.q[rows][:, c0 // 2:c1 // 2].contiguous()
        sf = nvfp4.swizzle_sf(sfb[rows][:, c0 // 16:c1 // 16].contiguous())
        wq = Nvfp4Tensor(q, sf, full.gscale, q.shape[0], c1 - c0)
        self = cls.from_nvfp4(wq, torch.tensor([8.0 / (6.0 * 448.0)], device=q.device), name=name)
        return self

    @classmethod
    def from_nvfp4(cls, wq: Nvfp4Tensor, input_scale: torch.Tensor, name: str = "") -> "Linear":
        """Wraps tensors loaded from a checkpoint (packed values, swizzled scales, weight_scale_2, input_scale)."""
        self = cls.__new__(cls)
        self.fmt, self.name, self.wq, self.weight = "nvfp4", name, wq, None
        self.out_features, self.in_features = wq.rows, wq.k
        self.calibrating, self.seen_amax, self.w3 = False, 0.0, None
        self.input_scale = input_scale.reshape(1).float()
        self.alpha = (self.input_scale * wq.gscale).reshape(1)
        return self

    def set_input_amax(self, amax: float) -> None:
        dev = self.wq.q.device
        self.input_scale = torch.tensor([max(amax, 1e-6) / (6.0 * 448.0)], dtype=torch.float32, device=dev)
        self.alpha = (self.input_scale * self.wq.gscale).reshape(1)

    def to(self, device) -> "Linear":
        if self.weight is not None:
            self.weight = self.weight.to(device)
        if self.wq is not None:
            w = self.wq
            self.wq = Nvfp4Tensor(w.q.to(device), w.sf.to(device), w.gscale.to(device), w.rows, w.k)
            self.input_scale = self.input_scale.to(device)
            self.alpha = self.alpha.to(device)
        return self

    def attach_w3(self) -> None:
        """Builds the 3-bit decode copy (int3, groups of 64, dequantisation fused into the GEMM) from this layer's
        served weights. Decode- and verify-sized calls then stream 4 bits per weight; prefill keeps the layer's own
        format. Reference: hibana/kernels/w3.py `attach_model` (HIBANA_W3_DECODE)."""
        from ..ops.w3gemm import W3Linear
        dev = self.weight.device if self.weight is not None else self.wq.q.device
        self.w3 = W3Linear.from_weight(self.dequantized(), dev, name=self.name + ".w3", keep_codes=dev.type != "cuda")

    def takes_w3(self, rows: int) -> bool:
        return self.w3 is not None and rows <= W3_MAX_ROWS and not self.calibrating

    def takes_gemv(self, rows: int) -> bool:
        """Up to eight bf16 rows against NVFP4 weights stream through the GEMV (ops/gemv.py): no activation
        quantisation, no tensor-memory or cluster state per launch. Off under `stable_numerics` (its results differ
        in the last bits from the GEMM's, so a request's tokens would depend on how many rows ran beside it)."""
        if self.fmt != "nvfp4" or self.calibrating or not self.wq.q.is_cuda:
            return False
        c = cfgmod.current()
        if not c.gemv or c.stable_numerics or self.out_features * self.in_features > GEMV_MAX_WEIGHTS:
            return False
        return 1 <= rows <= min(GEMV_MAX_ROWS, gemv.max_rows(self.out_features, self.in_features))

    def nbytes(self) -> int:
        if self.weight is not None:
            return self.weight.numel() * 2
        return self.wq.q.numel() + self.wq.sf.numel()

    def dequantized(self) -> torch.Tensor:
        return self.weight.float() if self.weight is not None else self.wq.dequantize()

    def quantize_input(self, x: torch.Tensor, mode: int = nvfp4.MODE_PLAIN) -> Activation:
        if self.fmt != "nvfp4":
            if mode != nvfp4.MODE_PLAIN:
                return basic.act_mul(x, basic.ACT_SILU_SPLIT if mode == nvfp4.MODE_SILU_SPLIT
                                     else basic.ACT_SILU_PAIRS)
            return x
        if self.calibrating:
            y = x if mode == nvfp4.MODE_PLAIN else nvfp4._silu_mul(x, mode)
            self.seen_amax = max(self.seen_amax, float(y.float().abs().max()))
        return nvfp4.quantize(x, self.input_scale, mode)

    def __call__(self, x: Activation, *, epilogue: int = gemm.EPI_STORE, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, requant: Optional[torch.Tensor] = None):
        """`requant` (the consuming projection's static input scale; SiLU-mul epilogue only): return the result as
        an Nvfp4Tensor, quantised inside the GEMM epilogue where the shape allows it."""
        if not isinstance(x, Nvfp4Tensor) and self.takes_w3(x.shape[0]):
            y = self.w3(x, epilogue=epilogue, residual=residual, out=out)
            return y if requant is None else nvfp4.quantize(y, requant)
        if self.fmt == "bf16":
            y = gemm.linear_bf16(x, self.weight, epilogue=epilogue, residual=residual, out=out)
            return y if requant is None else nvfp4.quantize(y, requant)
        if (not isinstance(x, Nvfp4Tensor) and epilogue in (gemm.EPI_STORE, gemm.EPI_RESIDUAL, gemm.EPI_SILU_MUL)
                and self.takes_gemv(x.shape[0])):
            y = gemv.nvfp4_gemv(x, self.wq, epilogue=epilogue, residual=residual, out=out)
            return y if requant is None else nvfp4.quantize(y, requant)
        xq = x if isinstance(x, Nvfp4Tensor) else self.quantize_input(x)
        if requant is not None and epilogue == gemm.EPI_SILU_MUL:
            return gemm.linear_nvfp4_silu_quant(xq, self.wq, self.alpha, requant)
        y = gemm.linear_nvfp4(xq, self.wq, self.alpha, epilogue=epilogue, residual=residual, out=out)
        return y if requant is None else nvfp4.quantize(y, requant)


def norm_linear(x: torch.Tensor, residual: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                lin: Linear, *, gemma: bool = False, epilogue: int = gemm.EPI_STORE,
                add_residual: bool = True, requant: Optional[torch.Tensor] = None):
    """lin(rmsnorm(x + residual)); `residual` is updated in place with the sum when add_residual."""
    res = residual if add_residual else None
    if lin.takes_w3(x.shape[0]):       # the 3-bit copy reads bf16 activations
        return lin(basic.rmsnorm(x, norm_weight, eps, residual=res, gemma=gemma), epilogue=epilogue, requant=requant)
    if lin.takes_gemv(x.shape[0]) and epilogue in (gemm.EPI_STORE, gemm.EPI_SILU_MUL):
        if res is not None:            # the sum has to land in the residual before any CTA normalises it
            y = lin(basic.rmsnorm(x, norm_weight, eps, residual=res, gemma=gemma), epilogue=epilogue)
        else:                          # the norm runs in the GEMV's prologue
            y = gemv.nvfp4_gemv(x, lin.wq, norm_weight=norm_weight, eps=eps, gemma=gemma, epilogue=epilogue)
        return y if requant is None else nvfp4.quantize(y, requant)
    if lin.fmt == "nvfp4":
        if lin.calibrating:
            y = basic.rmsnorm(x, norm_weight, eps, residual=res, gemma=gemma)
            lin.seen_amax = max(lin.seen_amax, float(y.float().abs().max()))
            return lin(nvfp4.quantize(y, lin.input_scale), epilogue=epilogue)
        xq, _ = nvfp4.rmsnorm_quantize(x, norm_weight, eps, lin.input_scale, residual=res, gemma=gemma)
        return lin(xq, epilogue=epilogue, requant=requant)
    y = basic.rmsnorm(x, norm_weight, eps, residual=res, gemma=gemma)
    return lin(y, epilogue=epilogue, requant=requant)
