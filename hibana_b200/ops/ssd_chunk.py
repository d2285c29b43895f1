"""Chunked (SSD) form of the Mamba-2 selective scan for prefill.

Per head, with a_t = dt_t * A the log decay, gamma its running sum inside a chunk of 64 tokens and L[t, i] =
exp(gamma_t - gamma_i) for i <= t:

    Y   = (L * (C B^T)) (dt * X)  +  (e^gamma * C) h0^T          h_C = e^gamma_C h0 + (e^(gamma_C - gamma) * B)^T (dt * X)

which is the chunk recurrence of the gated delta rule without its W term, so phase 2 is the same state-pass
kernel (csrc/gdn_chunk.cu, value dim = head dim, key dim = state dim 128) and phase 1 one kernel per (chunk, head)
(`ssd_phase1_kernel`; a handful of batched PyTorch products on the CPU path). The skip term D * x is added at the end. Only the fp32 state format takes this
path; quantised states keep the token-serial kernel. Reference: hibana/kernels/mamba2.py (chunked SSD prefill).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from .. import _native as nv
from .. import config as cfgmod
from . import gdn_chunk

CHUNK = gdn_chunk.CHUNK

P, I, L = nv.P, nv.I, nv.L
nv.register("hb_ssd_phase1", [P, P, P, P, P, P, L, L, L, I, I, I, I, P, P, P, P, P, P])


def prepare(x, bmat, cmat, dt, a_log, dt_bias, *, heads: int, groups: int, head_dim: int, d_state: int) -> dict:
    """Phase 1 for the rows of one sequence; tensors come back as [H, NC, C, *] fp32."""
    n = x.shape[0]
    nc = (n + CHUNK - 1) // CHUNK
    pad = nc * CHUNK - n
    hpg = heads // groups

    def chunks(t: torch.Tensor) -> torch.Tensor:          # [n, h, d] -> [h, nc, C, d], zero padded
        if pad:
            t = torch.cat([t, t.new_zeros(pad, *t.shape[1:])], 0)
        return t.view(nc, CHUNK, t.shape[1], -1).permute(2, 0, 1, 3)

    dtv = F.softplus(dt.float() + (dt_bias.float() if dt_bias is not None else 0.0))      # [n, H]
    a = -torch.exp(a_log.float())
    dtc = chunks(dtv.view(n, heads, 1)).squeeze(-1)                                       # [H, nc, C]; padding 0
    gam = (dtc * a[:, None, None]).cumsum(-1)
    diff = gam.unsqueeze(-1) - gam.unsqueeze(-2)
    low = torch.ones(CHUNK, CHUNK, dtype=torch.bool, device=x.device).tril()
    dec = torch.where(low, diff, diff.new_full((), float("-inf"))).exp()
    bc = chunks(bmat.float().view(n, groups, d_state))                                    # [G, nc, C, N]
    cc = chunks(cmat.float().view(n, groups, d_state))
    cb = (cc @ bc.transpose(-1, -2)).repeat_interleave(hpg, 0)                            # [H, nc, C, C]
    bh, ch = bc.repeat_interleave(hpg, 0), cc.repeat_interleave(hpg, 0)
    g_end = gam[..., -1]
    return {"u": dtc.unsqueeze(-1) * chunks(x.float().view(n, heads, head_dim)), "w": None, "m": cb * dec,
            "qg": ch * gam.exp().unsqueeze(-1), "kd": bh * (g_end[..., None] - gam).exp().unsqueeze(-1),
            "g_end": g_end, "n": n, "nc": nc}


def prepare_native(x, bmat, cmat, dt, a_log, dt_bias, *, heads: int, groups: int, head_dim: int) -> dict:
    """Phase 1 by csrc/gdn_chunk.cu (`ssd_phase1_kernel`): one CTA per (chunk, head); state dim 128."""
    n = x.shape[0]
    nc = (n + CHUNK - 1) // CHUNK
    dev, bf = x.device, torch.bfloat16
    out = {"w": None, "n": n, "nc": nc,
           "qg": torch.empty(heads, nc, CHUNK, 128, dtype=bf, device=dev),
           "kd": torch.empty(heads, nc, CHUNK, 128, dtype=bf, device=dev),
           "m": torch.empty(heads, nc, CHUNK, CHUNK, dtype=bf, device=dev),
           "u": torch.empty(heads, nc, CHUNK, head_dim, dtype=torch.float32, device=dev),
           "g_end": torch.empty(heads, nc, dtype=torch.float32, device=dev)}
    nv.check(nv.lib().hb_ssd_phase1(x.data_ptr(), bmat.data_ptr(), cmat.data_ptr(), dt.data_ptr(),
                                    a_log.data_ptr(), nv.ptr(dt_bias), x.stride(0), bmat.stride(0), dt.stride(0), n,
                                    heads, groups, head_dim, out["qg"].data_ptr(), out["kd"].data_ptr(),
                                    out["m"].data_ptr(), out["u"].data_ptr(), out["g_end"].data_ptr(), nv.stream()),
             "hb_ssd_phase1")
    return out


def mamba2_chunked(x, bmat, cmat, dt, a_log, dt_bias, dskip, state, slot_in, slot_out, *, heads: int, groups: int,
                   head_dim: int, d_state: int, ranges: Sequence[tuple[int, int]],
                   has_init: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Same contract as ops.recurrent.mamba2_scan for an fp32 state [slots, heads, P, N]."""
    y = torch.empty(x.shape[0], heads * head_dim, dtype=x.dtype, device=x.device)
    native = (nv.use_native(x) and d_state == 128 and head_dim % 32 == 0 and state.dtype == torch.float32
              and x.dtype == torch.bfloat16)
    sin = slot_in.tolist()
    sout = slot_out.tolist() if slot_out is not None else None
    for b, (r0, r1) in enumerate(ranges):
        if r1 <= r0:
            continue
        fused = (native and cfgmod.current().ssd_phase1 == "cuda" and dt.dtype == torch.bfloat16
                 and bmat.stride(0) == cmat.stride(0) and bmat.stride(0) % 4 == 0 and x.stride(0) % 2 == 0
                 and a_log.dtype == torch.float32 and (dt_bias is None or dt_bias.dtype == torch.float32))
        if fused:
            ph = prepare_native(x[r0:r1], bmat[r0:r1], cmat[r0:r1], dt[r0:r1], a_log, dt_bias, heads=heads,
                                groups=groups, head_dim=head_dim)
        else:
            ph = prepare(x[r0:r1], bmat[r0:r1], cmat[r0:r1], dt[r0:r1], a_log, dt_bias, heads=heads, groups=groups,
                         head_dim=head_dim, d_state=d_state)
        init = has_init is None or bool(has_init[b])
        if native:
            gdn_chunk._native_pass(ph, state[sin[b]] if init else None, state[sout[b]] if sout is not None else None,
                                   y[r0:r1], heads, d_state, head_dim)
        else:
            s0 = state[sin[b]] if init else torch.zeros_like(state[sin[b]])
            oc, s = gdn_chunk.state_pass_ref(ph, s0)
            n = r1 - r0
            y[r0:r1] = oc.permute(1, 2, 0, 3).reshape(ph["nc"] * CHUNK, heads * head_dim)[:n].to(y.dtype)
            if sout is not None:
                state[sout[b]] = s.to(state.dtype)
    if dskip is not None:
        y = (y.float() + dskip.float().repeat_interleave(head_dim)[None, :] * x.float()).to(x.dtype)
    return y
