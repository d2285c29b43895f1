"""FP8 (e4m3) linear layers: per-tensor weight scale, activations quantised with a static per-tensor scale or
dynamically per token (row amax / 448). The GEMM is the e4m3 kind of the tcgen05 kernel (csrc/gemm.cu,
tcgen05.mma kind::f8f6f4): small token counts put the weights on the 128-row side and split K over a cluster, so
the reference's separate CUDA-core GEMV for M <= 4 (hibana/kernels/csrc/fp8_gemv.cu) and its cuBLASLt path
(hibana/kernels/ops.py:95-128, hibana/model/flashnext/linear.py:77-133) are one kernel here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as nv
from . import gemm

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_quant_fp8_static", [P, L, P, P, P])
nv.register("hb_quant_fp8_rows", [P, I, I, P, P, P])
nv.register("hb_gemm_fp8", [P, P, I, I, I, L, L, P, L, P, Fl, P, P, I, I, I, P, I, P])

E4M3_MAX = 448.0


@dataclass
class Fp8Weight:
    q: torch.Tensor          # float8_e4m3fn [N, K]
    scale: torch.Tensor      # fp32 [1]: w ~= q * scale

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Fp8Weight":
        amax = float(w.float().abs().max().clamp_min(1e-12))
        scale = torch.tensor([amax / E4M3_MAX], dtype=torch.float32, device=w.device)
        return cls((w.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).contiguous(), scale)

    def dequantize(self) -> torch.Tensor:
        return self.q.float() * self.scale


def quantize_static(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """bf16 [.., K] -> e4m3 with one scale: q = x / scale (saturating)."""
    if nv.use_native(x):
        x = x.contiguous()
        q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        nv.check(nv.lib().hb_quant_fp8_static(x.data_ptr(), x.numel(), scale.data_ptr(), q.data_ptr(), nv.stream()),
                 "hb_quant_fp8_static")
        return q
    return (x.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def quantize_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [M, K] -> (e4m3 [M, K], fp32 scales [M]) with scale = row amax / 448."""
    m, k = x.shape
    if nv.use_native(x):
        x = x.contiguous()
        q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty(m, dtype=torch.float32, device=x.device)
        nv.check(nv.lib().hb_quant_fp8_rows(x.data_ptr(), m, k, q.data_ptr(), s.data_ptr(), nv.stream()),
                 "hb_quant_fp8_rows")
        return q, s
    s = (x.float().abs().amax(dim=1) / E4M3_MAX).clamp_min(1e-12)
    return (x.float() / s[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn), s


def linear_fp8(xq: torch.Tensor, w: Fp8Weight, *, x_scale: Optional[torch.Tensor] = None,
               row_scales: Optional[torch.Tensor] = None, epilogue: int = gemm.EPI_STORE,
               residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               splits: Optional[int] = None) -> torch.Tensor:
    """y = (xq * x_scale | xq * row_scales[:, None]) @ (w.q * w.scale).T for e4m3 xq [M, K]."""
    m, k = xq.shape
    n = w.q.shape[0]
    if not nv.use_native(xq, w.q):
        xf = xq.float() * (row_scales[:, None] if row_scales is not None else (x_scale if x_scale is not None else 1.0))
        res = gemm._ref_epilogue(xf @ w.dequantize().t(), epilogue, residual)
        if out is not None:
            out.copy_(res)
            return out
        return res
    out = gemm._out(m, n, epilogue, xq, out)
    swap, bn, auto_splits = gemm._plan(m, n, (k + 127) // 128, nv.WORKSPACE_BYTES)
    splits = auto_splits if splits is None else splits
    alpha_t = w.scale if x_scale is None else (w.scale * x_scale).reshape(1)
    st = nv.device_state(out.device)
    a, b, ra, rb = (w.q, xq, n, m) if swap else (xq, w.q, m, n)
    nv.check(nv.lib().hb_gemm_fp8(a.data_ptr(), b.data_ptr(), ra, rb, k, a.stride(0), b.stride(0), out.data_ptr(),
                                  out.stride(0), nv.ptr(residual), 1.0, alpha_t.data_ptr(), nv.ptr(row_scales),
                                  epilogue, int(swap), splits, st.status.data_ptr(), bn, nv.stream()), "hb_gemm_fp8")
    return out
