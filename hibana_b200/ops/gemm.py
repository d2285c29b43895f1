"""Linear layers on the tcgen05 GEMM (csrc/gemm.cu): bf16 and NVFP4, with fused epilogues.

Dispatch: up to 256 tokens the weight matrix takes the 128-row MMA operand ("swap") and K is split across
CTAs until the grid fills the 148 SMs, so a decode step streams every weight byte once at HBM rate; larger
token counts use 128 x 256 output tiles. The reference's equivalent dispatch (w3 -> verify GEMM -> tuned CUTLASS
tactic -> FlashInfer mm_fp4, and FP8 GEMV / cuBLASLt) is hibana/kernels/ops.py:56-128.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from .. import config as cfgmod
from .nvfp4 import Nvfp4Tensor

EPI_STORE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_STORE_F32 = 0, 1, 2, 3
EPI_SILU_MUL_QUANT = 7   # decode shapes (tokens <= 128): SiLU-mul, then NVFP4 requantisation in the same epilogue
EPI_RELU2 = 6       # grouped (weights on the 128-row side) GEMMs only: out = relu(x)^2
from ..hardware.b200 import NUM_SMS  # noqa: E402

nv.register("hb_gemm_set_pdl", [nv.I], void=True)
nv.register("hb_gemm_set_local_reduce", [nv.I], void=True)
nv.register("hb_gemm_silu_quant", [nv.I, nv.P, nv.P, nv.P, nv.P, nv.I, nv.I, nv.I, nv.L, nv.L, nv.P, nv.P, nv.P, nv.P,
                                   nv.I, nv.I, nv.P, nv.I, nv.I, nv.I, nv.P])
nv.register("hb_gemm_silu_quant_rows", [nv.I, nv.P, nv.P, nv.P, nv.P, nv.I, nv.I, nv.I, nv.L, nv.L, nv.P, nv.P, nv.P,
                                        nv.P, nv.I, nv.P, nv.I, nv.I, nv.I, nv.P])


_PDL_INIT = False


def set_pdl(on) -> None:
    """Programmatic dependent launch. Level 1 (True): GEMMs launch as dependents, their weight prefetch overlaps the
    kernel before them. Level 2: the small kernels of a decode step (quantisation, RoPE + KV write, decode
    attention, merge) do so too and GEMMs release their successor at their start. 0 / False: off."""
    global _PDL_INIT
    _PDL_INIT = True
    if nv.available():
        nv.lib().hb_gemm_set_pdl(int(on))
        nv.lib().hb_gemm_set_local_reduce(int(cfgmod.current().gemm_local_reduce))





def _plan(m: int, n: int, k_tiles: int, max_ws_bytes: int) -> tuple[bool, int, int]:
    """(swap, bn, splits) for an [m tokens] x [n features] problem."""
    if m <= 256:
        bn = next(b for b in (16, 32, 64, 128, 256) if b >= m)
        tiles = (n + 127) // 128
        splits = 1
        slots = NUM_SMS * (2 if bn <= 64 else 1)     # token tiles <= 64 run two CTAs per SM (csrc/gemm.cu Cfg)
        if cfgmod.current().stable_numerics:
            # the number of K splits (hence the order every output element is summed in) must not depend on how
            # many rows share the forward: a token then gets the same bits from a decode step, a verify round of
            # any depth and any batch (reference: hibana/kernels/stable.py, HIBANA_STABLE_NUMERICS)
            slots = NUM_SMS * 2
        if tiles < slots:
            # Fill the resident CTA slots without spilling into a second, mostly empty wave; every split keeps at
            # least two K tiles.
            splits = max(1, min(slots // tiles, k_tiles // 2, cfgmod.current().max_splits))
        return True, bn, splits
    return False, (256 if n >= 256 else 128), 1


def _launch(kind: int, a, b, sfa, sfb, ra: int, rb: int, k: int, lda: int, ldb: int, out: torch.Tensor,
            residual: Optional[torch.Tensor], alpha: float, alpha_ptr: Optional[torch.Tensor], epilogue: int,
            swap: bool, splits: int, bn: int, ka_a: int, ka_b: int) -> None:
    if not _PDL_INIT:
        set_pdl(cfgmod.current().pdl)
    st = nv.device_state(out.device)
    ws = cnt = None     # split-K reduces through distributed shared memory; no global scratch
    code = nv.lib().hb_gemm(kind, a.data_ptr(), b.data_ptr(), nv.ptr(sfa), nv.ptr(sfb), ra, rb, k, lda, ldb,
                            out.data_ptr(), out.stride(0), nv.ptr(residual), alpha, nv.ptr(alpha_ptr), epilogue,
                            int(swap), splits, nv.ptr(ws), nv.ptr(cnt), st.status.data_ptr(), bn, ka_a, ka_b,
                            nv.stream())
    nv.check(code, "hb_gemm")


def _out(m: int, n: int, epilogue: int, like: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
    cols = n // 2 if epilogue == EPI_SILU_MUL else n
    dtype = torch.float32 if epilogue == EPI_STORE_F32 else torch.bfloat16
    if out is None:
        out = torch.empty(m, cols, dtype=dtype, device=like.device)
    assert out.shape == (m, cols) and out.dtype == dtype and out.stride(1) == 1
    return out


def _ref_epilogue(acc: torch.Tensor, epilogue: int, residual: Optional[torch.Tensor]) -> torch.Tensor:
    if epilogue == EPI_RESIDUAL:
        return (acc + residual.float()).to(torch.bfloat16)
    if epilogue == EPI_SILU_MUL:
        return (torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]).to(torch.bfloat16)
    if epilogue == EPI_STORE_F32:
        return acc
    return acc.to(torch.bfloat16)


def linear_bf16(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_STORE, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, splits: Optional[int] = None) -> torch.Tensor:
    """y = x @ w.T for bf16 x [M, K], w [N, K] (fp32 accumulation)."""
    m, k = x.shape
    n = w.shape[0]
    if not nv.use_native(x, w):
        res = _ref_epilogue(x.float() @ w.float().t(), epilogue, residual)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    out = _out(m, n, epilogue, x, out)
    swap, bn, auto_splits = _plan(m, n, (k + 63) // 64, nv.WORKSPACE_BYTES)
    splits = auto_splits if splits is None else splits
    if swap:
        _launch(0, w, x, None, None, n, m, k, w.stride(0), x.stride(0), out, residual, 1.0, None, epilogue, True,
                splits, bn, 0, 0)
    else:
        _launch(0, x, w, None, None, m, n, k, x.stride(0), w.stride(0), out, residual, 1.0, None, epilogue, False,
                splits, bn, 0, 0)
    return out


def linear_nvfp4(x: Nvfp4Tensor, w: Nvfp4Tensor, alpha: torch.Tensor, *, epilogue: int = EPI_STORE,
                 residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 splits: Optional[int] = None) -> torch.Tensor:
    """y = dequant(x) @ dequant(w).T with block-scaled FP4 MMAs; `alpha` = x.gscale * w.gscale (device scalar)."""
    m, k, n = x.rows, x.k, w.rows
    assert w.k == k
    if not nv.use_native(x.q, w.q):
        acc = x.dequantize() @ w.dequantize().t()
        res = _ref_epilogue(acc, epilogue, residual)
        if out is not None:
            out.copy_(res)
            return out
        return res
    out = _out(m, n, epilogue, x.q, out)
    swap, bn, auto_splits = _plan(m, n, (k + 255) // 256, nv.WORKSPACE_BYTES)
    splits = auto_splits if splits is None else splits
    if swap:
        _launch(1, w.q, x.q, w.sf, x.sf, n, m, k, k, k, out, residual, 1.0, alpha, epilogue, True, splits, bn, w.ka,
                x.ka)
    else:
        _launch(1, x.q, w.q, x.sf, w.sf, m, n, k, k, k, out, residual, 1.0, alpha, epilogue, False, splits, bn, x.ka,
                w.ka)
    return out


_REQUANT_BUFS: dict = {}


def requant_ok(m: int, n: int) -> bool:
    """Shapes the fused SiLU-mul + requant epilogue covers: decode-sized calls with the weights on the 128-row side
    and whole feature tiles, and prefill-sized calls (tokens on the 128-row side, `_plan` picks that above 256 rows)
    whose feature count is a multiple of 64 (aligned 16-byte chunks of packed values)."""
    return (m <= 128 and n % 128 == 0) or (m > 256 and n % 64 == 0)


def linear_nvfp4_silu_quant(x: Nvfp4Tensor, w: Nvfp4Tensor, alpha: torch.Tensor, out_scale: torch.Tensor, *,
                            splits: Optional[int] = None) -> Nvfp4Tensor:
    """silu(gate) * up of y = x @ w.T (gate / up rows of `w` interleaved pairwise), requantised to NVFP4 with the
    static scale `out_scale` inside the GEMM epilogue: the result feeds the next NVFP4 projection directly.
    Bit-identical to `linear_nvfp4(..., epilogue=EPI_SILU_MUL)` followed by `nvfp4.quantize`.
    Reference: hibana/kernels/mlp_fusion.py:244-245."""
    from . import nvfp4
    m, k, n = x.rows, x.k, w.rows
    if not nv.use_native(x.q, w.q) or not requant_ok(m, n):
        return nvfp4.quantize(linear_nvfp4(x, w, alpha, epilogue=EPI_SILU_MUL), out_scale)
    ko = n // 2
    if m > 128:
        # prefill-sized: fresh buffers (chunk lengths vary and nothing here is captured); scale bytes the kernel
        # does not write (padding rows of the last 128-row block, padding groups of the last K atom) must read zero
        q, sf = nvfp4._alloc(m, ko, x.q.device)
        if m % 128 or ko % 64:
            sf.zero_()
        if not _PDL_INIT:
            set_pdl(cfgmod.current().pdl)
        st = nv.device_state(q.device)
        code = nv.lib().hb_gemm_silu_quant_rows(1, x.q.data_ptr(), w.q.data_ptr(), x.sf.data_ptr(), w.sf.data_ptr(),
                                                m, n, k, k, k, alpha.data_ptr(), q.data_ptr(), sf.data_ptr(),
                                                out_scale.data_ptr(), sf.shape[1], st.status.data_ptr(),
                                                256 if n >= 256 else 128, x.ka, w.ka, nv.stream())
        nv.check(code, "hb_gemm_silu_quant_rows")
        return Nvfp4Tensor(q, sf, out_scale, m, ko)
    key = (x.q.device, m, ko)
    bufs = _REQUANT_BUFS.get(key)
    if bufs is None:
        # persistent per shape (stable addresses inside captured graphs); scale bytes of padding rows and padding
        # groups are zeroed once, the kernel writes the real ones
        q, sf = nvfp4._alloc(m, ko, x.q.device)
        sf.zero_()
        bufs = _REQUANT_BUFS[key] = (q, sf)
    q, sf = bufs
    _, bn, auto_splits = _plan(m, n, (k + 255) // 256, nv.WORKSPACE_BYTES)
    if not _PDL_INIT:
        set_pdl(cfgmod.current().pdl)
    st = nv.device_state(q.device)
    code = nv.lib().hb_gemm_silu_quant(1, w.q.data_ptr(), x.q.data_ptr(), w.sf.data_ptr(), x.sf.data_ptr(), n, m, k,
                                       k, k, alpha.data_ptr(), q.data_ptr(), sf.data_ptr(), out_scale.data_ptr(),
                                       sf.shape[1], auto_splits if splits is None else splits,
                                       st.status.data_ptr(), bn, w.ka, x.ka, nv.stream())
    nv.check(code, "hb_gemm_silu_quant")
    return Nvfp4Tensor(q, sf, out_scale, m, ko)
