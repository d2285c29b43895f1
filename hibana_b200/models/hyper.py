"""Hyper-connections: `hc` residual streams per token, mixed into one block input and re-injected after the block.

    mix:     normed = per-stream Gemma RMSNorm(hyper)                        [T, hc, H]
             gate   = sigmoid(up(silu(down(normed) / hc)))                   [T, hc, H], low rank
             input  = mean over streams of gate * normed                     [T, H]
    combine: inject = 2 * sigmoid(inject_w(normed) / hc)                     [T, hc]
             hyper' = hyper + block_output[:, None, :] * inject[:, :, None]
The norm, the gated mean and the injection are single-pass CUDA kernels (csrc/hyper.cu); the three small
projections are tcgen05 GEMMs. Reference: hibana/model/flashnext/hyper.py:1-121, hibana/model/flashnext/model.py:42-77.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as nv
from ..ops import gemm

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_hc_norm", [P, P, P, I, I, I, Fl, P])
nv.register("hb_hc_gate_mean", [P, P, P, I, I, I, P])
nv.register("hb_hc_inject", [P, P, P, L, P, I, I, I, P])
nv.register("hb_hc_low", [P, L, P, I, I, P])


def grouped_norm_ref(hyper: torch.Tensor, w: torch.Tensor, hc: int, eps: float) -> torch.Tensor:
    t = hyper.shape[0]
    x = hyper.float().view(t, hc, -1)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + w.float().view(hc, -1))
    return y.view(t, -1).to(torch.bfloat16)


class HyperConnection:
    def __init__(self, norm: torch.Tensor, down: torch.Tensor, up: torch.Tensor, inject: torch.Tensor | None, hc: int,
                 hidden: int, eps: float = 1e-6):
        """norm [hc * H]; down [rank, hc * H]; up [hc * H, rank]; inject [hc, hc * H] (None on the last site)."""
        self.hc, self.hidden, self.eps = hc, hidden, eps
        self.norm = norm.to(torch.bfloat16).contiguous()
        self.down = (down / hc).to(torch.bfloat16).contiguous()          # the 1 / hc folded in (power of two: exact)
        self.up = up.to(torch.bfloat16).contiguous()
        inj = None
        if inject is not None:
            # the GEMM wants at least 16 output rows: pad the hc rows with zeros, read the first hc logits
            inj = torch.zeros(16, hc * hidden, dtype=torch.bfloat16, device=inject.device)
            inj[:hc] = (inject / hc).to(torch.bfloat16)
        self.inject = inj
        # one projection for both readers of the normed streams on the GPU: rows [down | inject] (the rank is padded
        # to a multiple of 16 rows by the inject block), fp32 out; `low` and the inject logits are cut from it
        self.rank = self.down.shape[0]
        self.down_inject = torch.cat((self.down, inj), 0).contiguous() if inj is not None else None

    def normed(self, hyper: torch.Tensor) -> torch.Tensor:
        t = hyper.shape[0]
        if not nv.use_native(hyper):
            return grouped_norm_ref(hyper, self.norm, self.hc, self.eps)
        out = torch.empty_like(hyper)
        nv.check(nv.lib().hb_hc_norm(hyper.data_ptr(), self.norm.data_ptr(), out.data_ptr(), t, self.hc, self.hidden,
                                     self.eps, nv.stream()), "hb_hc_norm")
        return out

    def mix(self, hyper: torch.Tensor):
        """hyper [T, hc * H] bf16 -> (block input [T, H], residuals for `combine`)."""
        t = hyper.shape[0]
        n = self.normed(hyper)
        both = None
        if nv.use_native(hyper) and self.down_inject is not None:
            both = gemm.linear_bf16(n, self.down_inject, epilogue=gemm.EPI_STORE_F32)      # [T, rank + 16] fp32
            low = torch.empty(t, self.rank, dtype=torch.bfloat16, device=hyper.device)
            nv.check(nv.lib().hb_hc_low(both.data_ptr(), both.stride(0), low.data_ptr(), t, self.rank, nv.stream()),
                     "hb_hc_low")
        else:
            low = F.silu(gemm.linear_bf16(n, self.down))    # one elementwise launch (fp32 math inside, bf16 out)
        gate = gemm.linear_bf16(low, self.up)
        if nv.use_native(hyper):
            mixed = torch.empty(t, self.hidden, dtype=torch.bfloat16, device=hyper.device)
            nv.check(nv.lib().hb_hc_gate_mean(gate.data_ptr(), n.data_ptr(), mixed.data_ptr(), t, self.hc, self.hidden,
                                              nv.stream()), "hb_hc_gate_mean")
        else:
            mixed = (torch.sigmoid(gate.float()).view(t, self.hc, -1) * n.float().view(t, self.hc, -1)).mean(1)
            mixed = mixed.to(torch.bfloat16)
        return mixed, (hyper, n, both)

    def combine(self, block_output: torch.Tensor, residuals) -> torch.Tensor:
        hyper, n, both = residuals
        t = hyper.shape[0]
        if both is not None:          # the inject logits came with the gate's first projection (mix)
            logits = both[:, self.rank:]
        else:
            logits = gemm.linear_bf16(n, self.inject, epilogue=gemm.EPI_STORE_F32)[:, :self.hc]
        if nv.use_native(hyper):
            out = torch.empty_like(hyper)
            nv.check(nv.lib().hb_hc_inject(hyper.data_ptr(), block_output.data_ptr(), logits.data_ptr(),
                                           logits.stride(0), out.data_ptr(), t, self.hc, self.hidden, nv.stream()),
                     "hb_hc_inject")
            return out
        inj = 2 * torch.sigmoid(logits.float())
        r = hyper.float().view(t, self.hc, -1) + block_output.float()[:, None, :] * inj[:, :, None]
        return r.view(t, -1).to(torch.bfloat16)
