"""NVFP4 weight-streaming GEMV for one to eight activation rows (csrc/gemv.cu).

`nvfp4_gemv(x, w)` is x @ dequant(w).T for bf16 `x` [M <= 8, K] against a served NVFP4 matrix, with the activations
left in bf16 (the tcgen05 GEMM quantises them to NVFP4 first). It exists for single-request decode and short
speculative verify blocks, where the tensor-core GEMM is bound by its per-launch state and not by the weight
stream. Optional fused steps: RMSNorm of `x` on the way in (`norm_weight`), the result added to a residual in place
(`EPI_RESIDUAL` with `out is residual`), SiLU-mul over interleaved gate / up rows (`EPI_SILU_MUL`).
The CPU form is the fp32 reference of the same arithmetic (normed rows rounded to bf16, dequantised weights).
Reference: hibana/kernels/ops.py:19-21 (the M <= 4 GEMV that replaces cuBLAS below 5 rows).
"""
from __future__ import annotations

from functools import lru_cache
from typing import Optional

import torch

from .. import _native as nv
from .gemm import EPI_RESIDUAL, EPI_SILU_MUL, EPI_STORE
from .nvfp4 import Nvfp4Tensor

P, I, F = nv.P, nv.I, nv.F
nv.register("hb_nvfp4_gemv", [P, P, P, I, I, I, P, I, I, P, F, I, P, I, P, I, I, P])
nv.register("hb_nvfp4_gemv_max_rows", [I, I])

MAX_ROWS = 8


@lru_cache(maxsize=None)
def max_rows(n: int, k: int) -> int:
    """Rows the kernel takes for an [n, k] matrix: 0 when the shape is not supported (n % 16, k % 256), fewer than 8
    when the activation rows of two resident CTAs would not fit in shared memory."""
    if n % 16 or k % 256:
        return 0
    if nv.available():
        return int(nv.lib().hb_nvfp4_gemv_max_rows(n, k))
    return min(MAX_ROWS, (100 * 1024 - 2048) // ((k + 16) * 2))


def nvfp4_gemv(x: torch.Tensor, w: Nvfp4Tensor, *, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
               gemma: bool = False, epilogue: int = EPI_STORE, residual: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    m, k = x.shape
    n = w.rows
    assert k == w.k and x.dtype == torch.bfloat16 and x.stride(1) == 1
    assert epilogue in (EPI_STORE, EPI_RESIDUAL, EPI_SILU_MUL)
    cols = n // 2 if epilogue == EPI_SILU_MUL else n
    if out is None:
        out = torch.empty(m, cols, dtype=torch.bfloat16, device=x.device)
    assert out.shape == (m, cols) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    if epilogue == EPI_RESIDUAL:
        assert residual is not None and residual.shape == (m, n) and residual.stride(1) == 1
    if nv.use_native(x, w.q):
        if not 1 <= m <= max_rows(n, k):
            raise ValueError(f"nvfp4_gemv takes 1..{max_rows(n, k)} rows of K = {k}, got {m}")
        nv.check(nv.lib().hb_nvfp4_gemv(
            w.q.data_ptr(), w.sf.data_ptr(), w.gscale.data_ptr(), n, k, w.ka, x.data_ptr(), x.stride(0), m,
            nv.ptr(norm_weight), float(eps), int(gemma), nv.ptr(residual),
            residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0),
            {EPI_STORE: 0, EPI_RESIDUAL: 1, EPI_SILU_MUL: 2}[epilogue], nv.stream()), "hb_nvfp4_gemv")
        return out
    out.copy_(nvfp4_gemv_ref(x, w, norm_weight=norm_weight, eps=eps, gemma=gemma, epilogue=epilogue,
                             residual=residual))
    return out


def nvfp4_gemv_ref(x: torch.Tensor, w: Nvfp4Tensor, *, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                   gemma: bool = False, epilogue: int = EPI_STORE,
                   residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    xf = x.float()
    if norm_weight is not None:
        nw = norm_weight.float() + (1.0 if gemma else 0.0)
        xf = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * nw).to(torch.bfloat16).float()
    acc = xf @ w.dequantize().to(xf.device).t()
    if epilogue == EPI_RESIDUAL:
        return (acc + residual.float()).to(torch.bfloat16)
    if epilogue == EPI_SILU_MUL:
        return (torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]).to(torch.bfloat16)
    return acc.to(torch.bfloat16)
