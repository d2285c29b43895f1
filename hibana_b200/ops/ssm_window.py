"""Mamba-2 state as a quantised window record (csrc/ssm_window.cu): int8 boundary state + the tokens committed since.

`WindowState` is one layer's view of the record tensors of a `StatePool` built with `window > 0`:
`z` int8 [slots, H, P, N], `zscale` fp32 [slots, H, P], `win_b` fp16 [slots, G, cap, N], `win_u` fp16 [slots, H, cap, P],
`win_c` fp32 [slots, H, cap], `win_len` int32 [slots, G]; cap = window + 16. `step` runs decode / verify / replay
rows (`commit=False`: nothing is written, which is all a speculative verify pass needs); `to_dense` / `from_dense`
convert to and from a plain fp32 state for prefill chunks, which run the fp32 kernels on a temporary state.
The CPU path below is the reference of the same arithmetic (fp16 records, fold when a committing call finds a full
window, int8 rows with amax / 127 scales).
Reference: hibana/cache/ssm_format.py:1-60, hibana/kernels/ssm_window.py:182-391.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as nv

P_, I, L = nv.P, nv.I, nv.L
nv.register("hb_mamba2_window", [P_, P_, P_, P_, L, L, L, P_, P_, P_, P_, L, P_, P_, P_, P_, P_, P_, P_, P_, P_,
                                 I, I, I, I, I, I, I, I, P_, P_])
nv.register("hb_window_delta_rule", [P_, P_, nv.F, I], void=True)
nv.register("hb_mamba2_window_io", [P_, P_, P_, P_, P_, P_, P_, P_, I, I, I, I, I, I, I, P_])

EXTRA = 16          # records a call may append beyond the window before the next committing call folds
MAX_ROWS = 16       # rows of one sequence per call


@dataclass
class WindowState:
    z: torch.Tensor
    zscale: torch.Tensor
    win_b: torch.Tensor
    win_u: torch.Tensor
    win_c: torch.Tensor
    win_len: torch.Tensor
    window: int

    @property
    def cap(self) -> int:
        return self.window + EXTRA

    @property
    def dims(self):
        _, h, p, n = self.z.shape
        return h, self.win_b.shape[1], p, n


def _fold_ref(ws: WindowState, slot: int, g: int, fresh: bool) -> None:
    """Folds group g's records of `slot` into a new boundary state (zeros when `fresh`)."""
    h, groups, p, n = ws.dims
    hg = h // groups
    ln = 0 if fresh else int(ws.win_len[slot, g])
    for hh in range(g * hg, (g + 1) * hg):
        if fresh:
            s = torch.zeros(p, n)
        else:
            c = ws.win_c[slot, hh, :ln]
            clast = c[-1] if ln else torch.tensor(0.0)
            s = torch.exp(clast) * ws.zscale[slot, hh][:, None] * ws.z[slot, hh].float()
            for j in range(ln):
                s = s + torch.exp(clast - c[j]) * ws.win_u[slot, hh, j].float()[:, None] * ws.win_b[slot, g, j].float()[None, :]
        amax = s.abs().amax(-1)
        inv = torch.where(amax > 0, 127.0 / amax, torch.zeros_like(amax))
        ws.z[slot, hh] = torch.round(s * inv[:, None]).clamp(-127, 127).to(torch.int8)
        ws.zscale[slot, hh] = amax / 127.0
    ws.win_len[slot, g] = 0


def step(ws: WindowState, x: torch.Tensor, bmat: torch.Tensor, cmat: torch.Tensor, dt: torch.Tensor,
         a_log: torch.Tensor, dt_bias: Optional[torch.Tensor], dskip: Optional[torch.Tensor], slots: torch.Tensor, *,
         q_indptr: Optional[torch.Tensor] = None, has_init: Optional[torch.Tensor] = None,
         commit: bool = True) -> torch.Tensor:
    """Rows of B sequences (one each, or `q_indptr` ranges of up to 16) against their window records. Returns
    y [T, H * P] bf16. `commit=False` reads only."""
    h, groups, p, n = ws.dims
    t = x.shape[0]
    batch = slots.shape[0]
    if nv.use_native(x, ws.z):
        y = torch.empty(t, h * p, dtype=torch.bfloat16, device=x.device)
        st = nv.device_state(x.device)
        nv.check(nv.lib().hb_mamba2_window(
            x.data_ptr(), bmat.data_ptr(), cmat.data_ptr(), dt.data_ptr(), x.stride(0), bmat.stride(0), dt.stride(0),
            a_log.data_ptr(), nv.ptr(dt_bias), nv.ptr(dskip), y.data_ptr(), y.stride(0), ws.z.data_ptr(),
            ws.zscale.data_ptr(), ws.win_b.data_ptr(), ws.win_u.data_ptr(), ws.win_c.data_ptr(), ws.win_len.data_ptr(),
            nv.ptr(q_indptr), slots.data_ptr(), nv.ptr(has_init), batch, h, groups, p, n, ws.window, ws.cap,
            int(commit), st.status.data_ptr(), nv.stream()), "hb_mamba2_window")
        return y
    hg = h // groups
    y = torch.empty(t, h * p, dtype=torch.bfloat16)
    a = -torch.exp(a_log.float())
    ip = q_indptr.tolist() if q_indptr is not None else list(range(batch + 1))
    for b in range(batch):
        slot = int(slots[b])
        fresh = has_init is not None and int(has_init[b]) == 0
        rows = range(ip[b], ip[b + 1])
        assert len(rows) <= MAX_ROWS
        for g in range(groups):
            ln = 0 if fresh else int(ws.win_len[slot, g])
            if commit and (ln >= ws.window or fresh):
                _fold_ref(ws, slot, g, fresh)
                ln = 0
            zs = torch.zeros(hg, p) if (fresh and not commit) else ws.zscale[slot, g * hg:(g + 1) * hg].clone()
            zq = ws.z[slot, g * hg:(g + 1) * hg].float()
            rec_b = [ws.win_b[slot, g, j].float() for j in range(ln)]
            rec_u = [ws.win_u[slot, g * hg:(g + 1) * hg, j].float() for j in range(ln)]          # [hg, p] each
            rec_c = [ws.win_c[slot, g * hg:(g + 1) * hg, j].clone() for j in range(ln)]          # [hg] each
            cum = rec_c[-1].clone() if ln else torch.zeros(hg)
            for r in rows:
                cv = cmat[r].float().view(groups, n)[g]
                bv = bmat[r].float().view(groups, n)[g].to(torch.float16).float()
                dtv = F.softplus(dt[r].float()[g * hg:(g + 1) * hg] + (dt_bias.float()[g * hg:(g + 1) * hg]
                                                                        if dt_bias is not None else 0.0))
                xv = x[r].float().view(h, p)[g * hg:(g + 1) * hg]
                cum = cum + dtv * a[g * hg:(g + 1) * hg]
                u = (dtv[:, None] * xv).to(torch.float16).float()
                rec_b.append(bv)
                rec_u.append(u)
                rec_c.append(cum.clone())
                out = torch.exp(cum)[:, None] * zs * (zq @ cv)
                for j in range(len(rec_b)):
                    out = out + (torch.exp(cum - rec_c[j]) * (rec_b[j] @ cv))[:, None] * rec_u[j]
                if dskip is not None:
                    out = out + dskip.float()[g * hg:(g + 1) * hg, None] * xv
                y[r].view(h, p)[g * hg:(g + 1) * hg] = out.to(torch.bfloat16)
                if commit:
                    j = len(rec_b) - 1
                    ws.win_b[slot, g, j] = bv.to(torch.float16)
                    ws.win_u[slot, g * hg:(g + 1) * hg, j] = u.to(torch.float16)
                    ws.win_c[slot, g * hg:(g + 1) * hg, j] = cum
            if commit:
                ws.win_len[slot, g] = len(rec_b)
    return y


def step_delta(ws: WindowState, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
               beta: torch.Tensor, slots: torch.Tensor, *, scale: Optional[float] = None, l2norm: bool = True,
               q_indptr: Optional[torch.Tensor] = None, has_init: Optional[torch.Tensor] = None,
               commit: bool = True) -> torch.Tensor:
    """The gated delta rule over the same record: heads = value heads, groups = key heads, a record is the row's
    (normalised, fp16) key, its correction u = beta (v - (decayed state) k) and the running log decay. q, k
    [T, key heads * K] (same row pitch), v [T, value heads * V] bf16; g, beta fp32 [T, value heads] contiguous."""
    h, groups, p, n = ws.dims
    t = q.shape[0]
    batch = slots.shape[0]
    scale = n ** -0.5 if scale is None else scale
    if nv.use_native(q, ws.z):
        assert q.stride(0) == k.stride(0) and g.is_contiguous() and beta.is_contiguous()
        y = torch.empty(t, h * p, dtype=torch.bfloat16, device=q.device)
        st = nv.device_state(q.device)
        lib = nv.lib()
        lib.hb_window_delta_rule(g.data_ptr(), beta.data_ptr(), float(scale), int(l2norm))
        nv.check(lib.hb_mamba2_window(
            v.data_ptr(), k.data_ptr(), q.data_ptr(), None, v.stride(0), k.stride(0), 0, None, None, None,
            y.data_ptr(), y.stride(0), ws.z.data_ptr(), ws.zscale.data_ptr(), ws.win_b.data_ptr(), ws.win_u.data_ptr(),
            ws.win_c.data_ptr(), ws.win_len.data_ptr(), nv.ptr(q_indptr), slots.data_ptr(), nv.ptr(has_init), batch, h,
            groups, p, n, ws.window, ws.cap, int(commit), st.status.data_ptr(), nv.stream()), "hb_mamba2_window")
        return y
    hg = h // groups
    y = torch.empty(t, h * p, dtype=torch.bfloat16)
    ip = q_indptr.tolist() if q_indptr is not None else list(range(batch + 1))
    for b in range(batch):
        slot = int(slots[b])
        fresh = has_init is not None and int(has_init[b]) == 0
        rows = range(ip[b], ip[b + 1])
        assert len(rows) <= MAX_ROWS
        for gi in range(groups):
            hs = slice(gi * hg, (gi + 1) * hg)
            ln = 0 if fresh else int(ws.win_len[slot, gi])
            if commit and (ln >= ws.window or fresh):
                _fold_ref(ws, slot, gi, fresh)
                ln = 0
            zs = torch.zeros(hg, p) if (fresh and not commit) else ws.zscale[slot, hs].clone()
            zq = ws.z[slot, hs].float()
            rec_k = [ws.win_b[slot, gi, j].float() for j in range(ln)]
            rec_u = [ws.win_u[slot, hs, j].float() for j in range(ln)]
            rec_c = [ws.win_c[slot, hs, j].clone() for j in range(ln)]
            cum = rec_c[-1].clone() if ln else torch.zeros(hg)
            for r in rows:
                qv = q[r].float().view(groups, n)[gi]
                kv = k[r].float().view(groups, n)[gi]
                if l2norm:
                    qv = qv * torch.rsqrt(qv.pow(2).sum() + 1e-6)
                    kv = kv * torch.rsqrt(kv.pow(2).sum() + 1e-6)
                qv = qv * scale
                kv = kv.to(torch.float16).float()
                vv = v[r].float().view(h, p)[hs]
                cum = cum + g[r].float()[hs]
                gain = torch.exp(cum)[:, None] * zs
                sk = gain * (zq @ kv)
                out = gain * (zq @ qv)
                for j in range(len(rec_k)):
                    dec = torch.exp(cum - rec_c[j])
                    sk = sk + (dec * (rec_k[j] @ kv))[:, None] * rec_u[j]
                    out = out + (dec * (rec_k[j] @ qv))[:, None] * rec_u[j]
                u = (beta[r].float()[hs][:, None] * (vv - sk)).to(torch.float16).float()
                out = out + (kv @ qv) * u
                rec_k.append(kv)
                rec_u.append(u)
                rec_c.append(cum.clone())
                y[r].view(h, p)[hs] = out.to(torch.bfloat16)
                if commit:
                    j = len(rec_k) - 1
                    ws.win_b[slot, gi, j] = kv.to(torch.float16)
                    ws.win_u[slot, hs, j] = u.to(torch.float16)
                    ws.win_c[slot, hs, j] = cum
            if commit:
                ws.win_len[slot, gi] = len(rec_k)
    return y


def to_dense(ws: WindowState, slots: torch.Tensor) -> torch.Tensor:
    """fp32 [B, H, P, N]: the states the records of `slots` stand for."""
    h, groups, p, n = ws.dims
    b = slots.shape[0]
    if nv.use_native(ws.z):
        out = torch.empty(b, h, p, n, dtype=torch.float32, device=ws.z.device)
        nv.check(nv.lib().hb_mamba2_window_io(out.data_ptr(), ws.z.data_ptr(), ws.zscale.data_ptr(), ws.win_b.data_ptr(),
                                              ws.win_u.data_ptr(), ws.win_c.data_ptr(), ws.win_len.data_ptr(),
                                              slots.data_ptr(), b, h, groups, p, n, ws.cap, 1, nv.stream()),
                 "hb_mamba2_window_io")
        return out
    hg = h // groups
    out = torch.zeros(b, h, p, n)
    for i in range(b):
        slot = int(slots[i])
        for hh in range(h):
            g = hh // hg
            ln = int(ws.win_len[slot, g])
            c = ws.win_c[slot, hh, :ln]
            clast = c[-1] if ln else torch.tensor(0.0)
            s = torch.exp(clast) * ws.zscale[slot, hh][:, None] * ws.z[slot, hh].float()
            for j in range(ln):
                s = s + torch.exp(clast - c[j]) * ws.win_u[slot, hh, j].float()[:, None] * ws.win_b[slot, g, j].float()[None, :]
            out[i, hh] = s
    return out


def from_dense(ws: WindowState, slots: torch.Tensor, dense: torch.Tensor) -> None:
    """The records of `slots` become fresh boundary states quantised from dense [B, H, P, N] fp32."""
    h, groups, p, n = ws.dims
    b = slots.shape[0]
    if nv.use_native(ws.z):
        dense = dense.contiguous()
        nv.check(nv.lib().hb_mamba2_window_io(dense.data_ptr(), ws.z.data_ptr(), ws.zscale.data_ptr(), ws.win_b.data_ptr(),
                                              ws.win_u.data_ptr(), ws.win_c.data_ptr(), ws.win_len.data_ptr(),
                                              slots.data_ptr(), b, h, groups, p, n, ws.cap, 0, nv.stream()),
                 "hb_mamba2_window_io")
        return
    for i in range(b):
        slot = int(slots[i])
        s = dense[i].float()
        amax = s.abs().amax(-1)
        inv = torch.where(amax > 0, 127.0 / amax, torch.zeros_like(amax))
        ws.z[slot] = torch.round(s * inv[..., None]).clamp(-127, 127).to(torch.int8)
        ws.zscale[slot] = amax / 127.0
        ws.win_len[slot] = 0
