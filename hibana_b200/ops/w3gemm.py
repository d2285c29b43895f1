"""Linear layers on the 3-bit weight copy: y = x @ dequant(w3).T with the dequantisation fused into the tcgen05 GEMM
(csrc/gemm.cu kind w3). Decode / verify sized batches (up to 256 tokens) stream 4 bits per weight from HBM; larger
batches expand the matrix to bf16 once and use the bf16 GEMM (prefill is compute-bound, so the narrow copy buys
nothing there). Reference: hibana/kernels/w3.py:262-412 (dispatch, split table), hibana/kernels/csrc/w3_gemm.cu:114-640.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from ..weights.w3 import Int3G64
from . import gemm

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_gemm_w3", [P, P, I, I, I, L, P, L, P, Fl, I, I, P, I, P])


class W3Linear:
    def __init__(self, w3: Int3G64, device="cpu", name: str = "", keep_codes: bool = True):
        """`keep_codes=False`: drop the unpacked codes once the kernel's tiles exist (a byte per weight that only the
        reference path and `dense()` read); such a layer serves rows <= 256 on the GPU only."""
        self.w3, self.name = w3, name
        self.out_features, self.in_features = w3.shape
        self.device = torch.device(device)
        self.tiles = w3.tiles().to(self.device) if self.device.type == "cuda" else None
        self._dense: Optional[torch.Tensor] = None
        if not keep_codes and self.tiles is not None:
            self.w3 = None

    @classmethod
    def from_weight(cls, w: torch.Tensor, device="cpu", name: str = "", keep_codes: bool = True) -> "W3Linear":
        """Quantises on the device the weight is on (the big matrices of a 27B model never visit the host)."""
        src = w if w.is_cuda else w.cpu()
        return cls(Int3G64.quantize(src), device, name, keep_codes)

    def dense(self) -> torch.Tensor:
        if self._dense is None and self.w3 is None:
            raise RuntimeError("this 3-bit copy kept only its kernel tiles: it serves decode-sized calls on the GPU")
        if self._dense is None:
            self._dense = self.w3.dequantize().to(torch.bfloat16).to(self.device)
        return self._dense

    def nbytes(self) -> int:
        return self.tiles.numel() if self.tiles is not None else self.out_features * self.in_features // 2

    def __call__(self, x: torch.Tensor, *, epilogue: int = gemm.EPI_STORE, residual: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m, k = x.shape
        n = self.out_features
        if not nv.use_native(x) or m > 256:
            return gemm.linear_bf16(x, self.dense(), epilogue=epilogue, residual=residual, out=out)
        out = gemm._out(m, n, epilogue, x, out)
        _swap, bn, splits = gemm._plan(m, n, k // 64, nv.WORKSPACE_BYTES)
        st = nv.device_state(out.device)
        nv.check(nv.lib().hb_gemm_w3(self.tiles.data_ptr(), x.data_ptr(), n, m, k, x.stride(0), out.data_ptr(),
                                     out.stride(0), nv.ptr(residual), 1.0, epilogue, splits, st.status.data_ptr(), bn,
                                     nv.stream()), "hb_gemm_w3")
        return out
