"""Chunked (WY) form of the gated delta rule for prefill.

The recurrence  S <- e^g S ; v' = beta (v - S k) ; S <- S + v' k^T ; o = S q  is sequential in the token, but
within a chunk of C tokens everything except the dependence on the incoming state S0 can be computed for all
chunks at once. With gamma_t the running sum of g inside the chunk and D[t, i] = exp(gamma_t - gamma_i):

    A  = strict_lower(beta_t D[t, i] (k_t . k_i))            T = (I + A)^-1            (unit lower triangular)
    U  = T (beta * V)          W = T (beta * e^gamma * K)     V' = U - W S0^T
    O  = (e^gamma * Q) S0^T + lower(D * Q K^T) V'             S_C = e^gamma_C S0 + V'^T (e^(gamma_C - gamma) * K)

Phase 1 (all chunks and heads in parallel: `gdn_phase1_kernel` on the GPU for head dim 128, batched GEMMs and one
triangular solve in PyTorch otherwise) produces U, W, the masked
score matrix and the decayed Q / K; phase 2 walks the chunks of a sequence carrying S (three small products per
chunk; csrc/gdn_chunk.cu on the GPU, `state_pass_ref` here). Padding rows of the last chunk carry g = 0 and
beta = 0, which leaves the state untouched. Reference: hibana/kernels/fla/chunk.py (chunk_gated_delta_rule),
hibana/kernels/fla/wy_fast.py, hibana/kernels/fla/chunk_delta_h.py.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _native as nv
from .. import config as cfgmod

P, I, L = nv.P, nv.I, nv.L
nv.register("hb_gdn_chunk_pass", [P, P, P, P, P, P, P, P, P, L, I, I, I, I, I, P])
nv.register("hb_gdn_phase1", [P, P, P, P, P, L, L, I, I, I, nv.F, I, P, P, P, P, P, P, P])

CHUNK = 64


def prepare(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, *, k_heads: int,
            v_heads: int, kdim: int, vdim: int, scale: float, l2norm: bool, chunk: int = CHUNK) -> dict:
    """Phase 1 for the rows of ONE sequence. q, k [n, k_heads*K]; v [n, v_heads*V]; g, beta [n, v_heads].
    Returns fp32 tensors shaped [H, NC, C, *] (H = v_heads) and gC [H, NC]."""
    n = q.shape[0]
    rep = v_heads // k_heads
    nc = (n + chunk - 1) // chunk
    pad = nc * chunk - n
    qf = q.float().view(n, k_heads, kdim)
    kf = k.float().view(n, k_heads, kdim)
    if l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = qf * scale

    def chunks(x: torch.Tensor) -> torch.Tensor:          # [n, h, d] -> [h, nc, C, d], zero padded
        if pad:
            x = torch.cat([x, x.new_zeros(pad, *x.shape[1:])], 0)
        return x.view(nc, chunk, x.shape[1], -1).permute(2, 0, 1, 3)

    qc, kc = chunks(qf), chunks(kf)                        # [k_heads, nc, C, K]
    vc = chunks(v.float().view(n, v_heads, vdim))          # [H, nc, C, V]
    gc = chunks(g.float().view(n, v_heads, 1)).squeeze(-1)     # [H, nc, C]
    bc = chunks(beta.float().view(n, v_heads, 1)).squeeze(-1)
    gam = gc.cumsum(-1)
    diff = gam.unsqueeze(-1) - gam.unsqueeze(-2)           # gamma_t - gamma_i
    low = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    dec = torch.where(low, diff, diff.new_full((), float("-inf"))).exp()     # D, zero above the diagonal
    kk = (kc @ kc.transpose(-1, -2)).repeat_interleave(rep, 0)               # [H, nc, C, C]
    qk = (qc @ kc.transpose(-1, -2)).repeat_interleave(rep, 0)
    a = (bc.unsqueeze(-1) * dec * kk).tril(-1)
    eye = torch.eye(chunk, dtype=torch.float32, device=q.device)
    t = torch.linalg.solve_triangular(a + eye, eye.expand_as(a).contiguous(), upper=False)
    kh = kc.repeat_interleave(rep, 0)                      # [H, nc, C, K]
    qh = qc.repeat_interleave(rep, 0)
    eg = gam.exp().unsqueeze(-1)
    u = t @ (bc.unsqueeze(-1) * vc)
    w = t @ (bc.unsqueeze(-1) * eg * kh)
    g_end = gam[..., -1]
    return {"u": u, "w": w, "m": qk * dec, "qg": qh * eg, "kd": kh * (g_end[..., None] - gam).exp().unsqueeze(-1),
            "g_end": g_end, "n": n, "nc": nc}


def state_pass_ref(ph: dict, s0: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Phase 2 in PyTorch: returns (o [H, nc, C, V], final state [H, V, K])."""
    s = s0.float().clone()
    outs = []
    for c in range(ph["nc"]):
        st = s.transpose(1, 2)                             # [H, K, V]
        vn = ph["u"][:, c] - ph["w"][:, c] @ st if ph.get("w") is not None else ph["u"][:, c]
        outs.append(ph["qg"][:, c] @ st + ph["m"][:, c] @ vn)
        s = ph["g_end"][:, c].exp()[:, None, None] * s + vn.transpose(1, 2) @ ph["kd"][:, c]
    return torch.stack(outs, 1), s


def _native_pass(ph: dict, s_in: Optional[torch.Tensor], s_out: Optional[torch.Tensor], o_rows: torch.Tensor,
                 heads: int, kdim: int, vdim: int) -> None:
    """Phase 2 by csrc/gdn_chunk.cu: writes the sequence's output rows and the final state in place."""
    bf = torch.bfloat16
    qg, kd, m = (ph[name].to(bf).contiguous() for name in ("qg", "kd", "m"))
    w = ph["w"].to(bf).contiguous() if ph.get("w") is not None else None     # None: V' = U (Mamba-2 / SSD)
    u, g_end = ph["u"].contiguous(), ph["g_end"].contiguous()
    nv.check(nv.lib().hb_gdn_chunk_pass(nv.ptr(w), qg.data_ptr(), kd.data_ptr(), m.data_ptr(), u.data_ptr(),
                                        g_end.data_ptr(), nv.ptr(s_in), nv.ptr(s_out), o_rows.data_ptr(),
                                        o_rows.stride(0), heads, ph["nc"], ph["n"], kdim, vdim, nv.stream()),
             "hb_gdn_chunk_pass")


def prepare_native(q, k, v, g, beta, *, k_heads: int, v_heads: int, scale: float, l2norm: bool) -> dict:
    """Phase 1 by csrc/gdn_chunk.cu (`gdn_phase1_kernel`): one CTA per (chunk, head); key / value dim 128."""
    n = q.shape[0]
    nc = (n + CHUNK - 1) // CHUNK
    dev, bf = q.device, torch.bfloat16
    out = {name: torch.empty(v_heads, nc, CHUNK, 128, dtype=bf, device=dev) for name in ("w", "qg", "kd")}
    out["m"] = torch.empty(v_heads, nc, CHUNK, CHUNK, dtype=bf, device=dev)
    out["u"] = torch.empty(v_heads, nc, CHUNK, 128, dtype=torch.float32, device=dev)
    out["g_end"] = torch.empty(v_heads, nc, dtype=torch.float32, device=dev)
    out.update(n=n, nc=nc)
    nv.check(nv.lib().hb_gdn_phase1(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                    q.stride(0), v.stride(0), n, k_heads, v_heads, scale, int(l2norm),
                                    out["w"].data_ptr(), out["qg"].data_ptr(), out["kd"].data_ptr(),
                                    out["m"].data_ptr(), out["u"].data_ptr(), out["g_end"].data_ptr(), nv.stream()),
             "hb_gdn_phase1")
    return out


def gdn_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                state: torch.Tensor, slot_in: torch.Tensor, slot_out: Optional[torch.Tensor], *, k_heads: int,
                v_heads: int, kdim: int, vdim: int, scale: float, l2norm: bool,
                ranges: Sequence[tuple[int, int]], has_init: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Same contract as ops.recurrent.gdn_scan; `ranges` are the (first, last + 1) rows of each sequence."""
    o = torch.empty(q.shape[0], v_heads * vdim, dtype=q.dtype, device=q.device)
    native = (nv.use_native(q) and kdim == 128 and vdim == 128 and state.dtype == torch.float32
              and q.dtype == torch.bfloat16)
    sin = slot_in.tolist()
    sout = slot_out.tolist() if slot_out is not None else None
    for b, (r0, r1) in enumerate(ranges):
        if r1 <= r0:
            continue
        fused = (native and cfgmod.current().gdn_phase1 == "cuda" and q.stride(0) == k.stride(0)
                 and q.stride(0) % 4 == 0 and v.stride(0) % 4 == 0 and g.is_contiguous() and beta.is_contiguous())
        if fused:
            ph = prepare_native(q[r0:r1], k[r0:r1], v[r0:r1], g[r0:r1], beta[r0:r1], k_heads=k_heads,
                                v_heads=v_heads, scale=scale, l2norm=l2norm)
        else:
            ph = prepare(q[r0:r1], k[r0:r1], v[r0:r1], g[r0:r1], beta[r0:r1], k_heads=k_heads, v_heads=v_heads,
                         kdim=kdim, vdim=vdim, scale=scale, l2norm=l2norm)
        init = has_init is None or bool(has_init[b])
        if native:
            _native_pass(ph, state[sin[b]] if init else None, state[sout[b]] if sout is not None else None,
                         o[r0:r1], v_heads, kdim, vdim)
            continue
        s0 = state[sin[b]] if init else torch.zeros_like(state[sin[b]])
        oc, s = state_pass_ref(ph, s0)
        n = r1 - r0
        o[r0:r1] = oc.permute(1, 2, 0, 3).reshape(ph["nc"] * CHUNK, v_heads * vdim)[:n].to(o.dtype)
        if sout is not None:
            state[sout[b]] = s.to(state.dtype)
    return o
