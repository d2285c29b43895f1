"""Recurrent-layer ops: causal conv1d, Mamba-2 selective scan, gated delta rule (csrc/ssm.cu).

Each op is ragged (rows q_indptr[b]..q_indptr[b+1] belong to sequence b; None = one row each) and carries state
through pool slots: it reads `slot_in[b]` (unless has_init[b] == 0) and writes `slot_out[b]` (None = do not
write: verify). The PyTorch implementations are the fp32 sequential references and the CPU path.
Reference: hibana/kernels/mamba2.py, hibana/kernels/fla/*, hibana/kernels/csrc/gdn_verify.cu.
"""
from __future__ import annotations

import ctypes

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from .. import _native as nv

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_conv1d", [P, L, P, P, P, L, P, L, P, P, P, P, I, I, I, I, I, P])
nv.register("hb_mamba2_scan", [P, P, P, P, L, L, L, P, P, P, P, L, P, L, P, P, P, P, I, I, I, I, I, P])
nv.register("hb_mamba2_scan_fmt", [P, P, P, P, L, L, L, P, P, P, P, L, P, L, P, P, P, P, I, I, I, I, I, I, P, ctypes.c_uint, P])
nv.register("hb_gdn_scan", [P, P, P, P, P, L, L, P, L, P, L, P, P, P, P, I, I, I, I, I, Fl, I, P])


CHUNKED_MIN_ROWS = 128      # prefill chunks at least this long use the chunked gated delta rule


def _ranges(q_indptr, batch):
    if q_indptr is None:
        return [(b, b + 1) for b in range(batch)]
    ip = q_indptr.tolist()
    return [(ip[b], ip[b + 1]) for b in range(batch)]


def conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
           slot_in: torch.Tensor, slot_out: Optional[torch.Tensor], *, q_indptr: Optional[torch.Tensor] = None,
           has_init: Optional[torch.Tensor] = None, silu: bool = True, max_rows: int = 0) -> torch.Tensor:
    """x [T, C] bf16 (may be a column slice), weight [C, W], state [slots, C, W-1] bf16 (raw inputs). `max_rows`
    (host bound on rows per sequence; 0 = unknown) lets prefill chunks run parallel over tiles of tokens."""
    t, c = x.shape
    w = weight.shape[1]
    batch = slot_in.shape[0]
    if nv.use_native(x):
        y = torch.empty(t, c, dtype=x.dtype, device=x.device)
        nv.check(nv.lib().hb_conv1d(x.data_ptr(), x.stride(0), weight.data_ptr(), nv.ptr(bias), y.data_ptr(),
                                    y.stride(0), state.data_ptr(), state.stride(0), nv.ptr(q_indptr),
                                    slot_in.data_ptr(), nv.ptr(slot_out), nv.ptr(has_init), batch, c, w, int(silu),
                                    int(max_rows), nv.stream()), "hb_conv1d", launches=2 if max_rows > 32 else 1)
        return y
    y = torch.empty(t, c, dtype=x.dtype)
    wf = weight.float()
    for b, (r0, r1) in enumerate(_ranges(q_indptr, batch)):
        init = has_init is None or bool(has_init[b])
        win = state[int(slot_in[b])].float().t() if init else torch.zeros(w - 1, c)   # [W-1, C]
        seq = torch.cat([win, x[r0:r1].float()], dim=0)                                  # [W-1+n, C]
        n = r1 - r0
        acc = torch.zeros(n, c) + (bias.float() if bias is not None else 0.0)
        for j in range(w):
            acc = acc + seq[j:j + n] * wf[:, j]
        y[r0:r1] = (F.silu(acc) if silu else acc).to(x.dtype)
        if slot_out is not None:
            state[int(slot_out[b])] = seq[n:n + w - 1].t().to(state.dtype)
    return y


def mamba2_scan(x: torch.Tensor, bmat: torch.Tensor, cmat: torch.Tensor, dt: torch.Tensor, a_log: torch.Tensor,
                dt_bias: Optional[torch.Tensor], dskip: Optional[torch.Tensor], state: torch.Tensor,
                slot_in: torch.Tensor, slot_out: Optional[torch.Tensor], *, heads: int, groups: int, head_dim: int,
                d_state: int, q_indptr: Optional[torch.Tensor] = None,
                has_init: Optional[torch.Tensor] = None, state_scale: Optional[torch.Tensor] = None,
                sr_seed: int = 0, host_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """x [T, heads*P], bmat/cmat [T, groups*N], dt [T, heads] (bf16, column slices allowed);
    state [slots, heads, P, N] in fp32, fp16 (`sr_seed` != 0: stochastic rounding when the state is written back)
    or int8 with `state_scale` [slots, heads, P] fp32 row scales. Returns y [T, heads*P] bf16."""
    t = x.shape[0]
    batch = slot_in.shape[0]
    fmt = {torch.float32: 0, torch.float16: 1, torch.int8: 2}[state.dtype]
    if (nv.use_native(x) and fmt == 0 and d_state == 128 and host_rows is not None
            and max(host_rows) >= CHUNKED_MIN_ROWS):
        # long prefill chunks: the chunked (SSD) form, parallel over 64-token chunks (ops/ssd_chunk.py)
        from . import ssd_chunk
        ranges, r = [], 0
        for n in host_rows:
            ranges.append((r, r + n))
            r += n
        return ssd_chunk.mamba2_chunked(x, bmat, cmat, dt, a_log, dt_bias, dskip, state, slot_in, slot_out,
                                        heads=heads, groups=groups, head_dim=head_dim, d_state=d_state,
                                        ranges=ranges, has_init=None if has_init is None else has_init.tolist())
    if nv.use_native(x):
        y = torch.empty(t, heads * head_dim, dtype=x.dtype, device=x.device)
        nv.check(nv.lib().hb_mamba2_scan_fmt(
            x.data_ptr(), bmat.data_ptr(), cmat.data_ptr(), dt.data_ptr(), x.stride(0), bmat.stride(0), dt.stride(0),
            a_log.data_ptr(), nv.ptr(dt_bias), nv.ptr(dskip), y.data_ptr(), y.stride(0), state.data_ptr(),
            state.stride(0), nv.ptr(q_indptr), slot_in.data_ptr(), nv.ptr(slot_out), nv.ptr(has_init), batch, heads,
            groups, head_dim, d_state, fmt, nv.ptr(state_scale), sr_seed & 0xFFFFFFFF, nv.stream()),
                 "hb_mamba2_scan_fmt")
        return y
    if fmt != 0:      # CPU reference: dequantise the slots in use, run in fp32, requantise (round to nearest)
        work = torch.zeros(state.shape, dtype=torch.float32)
        used = torch.cat([slot_in.long(), slot_out.long() if slot_out is not None else slot_in.long()]).unique()
        deq = state[used].float() * (state_scale[used][..., None] if fmt == 2 else 1.0)
        work[used] = deq
        y = mamba2_scan(x, bmat, cmat, dt, a_log, dt_bias, dskip, work, slot_in, slot_out, heads=heads, groups=groups,
                        head_dim=head_dim, d_state=d_state, q_indptr=q_indptr, has_init=has_init)
        if slot_out is not None:
            for s_ in slot_out.long().unique().tolist():
                if fmt == 1:
                    state[s_] = work[s_].to(torch.float16)
                else:
                    sc = (work[s_].abs().amax(-1) / 127.0)
                    sc = torch.where(sc > 0, sc, torch.ones_like(sc))
                    state_scale[s_] = sc
                    state[s_] = torch.round(work[s_] / sc[..., None]).clamp(-127, 127).to(torch.int8)
        return y
    y = torch.empty(t, heads * head_dim, dtype=x.dtype)
    a = -torch.exp(a_log.float())
    hpg = heads // groups
    for b, (r0, r1) in enumerate(_ranges(q_indptr, batch)):
        init = has_init is None or bool(has_init[b])
        s = state[int(slot_in[b])].float().clone() if init else torch.zeros(heads, head_dim, d_state)
        for r in range(r0, r1):
            dtv = F.softplus(dt[r].float() + (dt_bias.float() if dt_bias is not None else 0.0))      # [heads]
            xv = x[r].float().view(heads, head_dim)
            bv = bmat[r].float().view(groups, d_state).repeat_interleave(hpg, 0)                      # [heads, N]
            cv = cmat[r].float().view(groups, d_state).repeat_interleave(hpg, 0)
            s = s * torch.exp(dtv * a)[:, None, None] + (dtv[:, None] * xv)[:, :, None] * bv[:, None, :]
            out = (s * cv[:, None, :]).sum(-1)
            if dskip is not None:
                out = out + dskip.float()[:, None] * xv
            y[r] = out.reshape(-1).to(x.dtype)
        if slot_out is not None:
            state[int(slot_out[b])] = s
    return y


def gdn_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
             state: torch.Tensor, slot_in: torch.Tensor, slot_out: Optional[torch.Tensor], *, k_heads: int,
             v_heads: int, kdim: int, vdim: int, scale: Optional[float] = None, l2norm: bool = True,
             q_indptr: Optional[torch.Tensor] = None, has_init: Optional[torch.Tensor] = None,
             host_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Gated delta rule. q, k [T, k_heads*K] (same row pitch), v [T, v_heads*V] bf16; g (log decay), beta
    [T, v_heads] fp32 contiguous; state [slots, v_heads, V, K] fp32. Returns o [T, v_heads*V] bf16.
    `host_rows` (rows per sequence, known on the host during prefill) lets long sequences take the chunked form
    (ops/gdn_chunk.py): tensor-core work parallel over chunks instead of one serial step per token."""
    t = q.shape[0]
    batch = slot_in.shape[0]
    scale = kdim ** -0.5 if scale is None else scale
    if nv.use_native(q) and host_rows is not None and max(host_rows) >= CHUNKED_MIN_ROWS:
        from . import gdn_chunk
        ranges, r = [], 0
        for n in host_rows:
            ranges.append((r, r + n))
            r += n
        return gdn_chunk.gdn_chunked(q, k, v, g, beta, state, slot_in, slot_out, k_heads=k_heads, v_heads=v_heads,
                                     kdim=kdim, vdim=vdim, scale=scale, l2norm=l2norm, ranges=ranges,
                                     has_init=None if has_init is None else has_init.tolist())
    if nv.use_native(q):
        assert q.stride(0) == k.stride(0) and g.is_contiguous() and beta.is_contiguous()
        o = torch.empty(t, v_heads * vdim, dtype=q.dtype, device=q.device)
        nv.check(nv.lib().hb_gdn_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                      q.stride(0), v.stride(0), o.data_ptr(), o.stride(0), state.data_ptr(),
                                      state.stride(0), nv.ptr(q_indptr), slot_in.data_ptr(), nv.ptr(slot_out),
                                      nv.ptr(has_init), batch, k_heads, v_heads, kdim, vdim, scale, int(l2norm),
                                      nv.stream()), "hb_gdn_scan")
        return o
    o = torch.empty(t, v_heads * vdim, dtype=q.dtype)
    rep = v_heads // k_heads
    for b, (r0, r1) in enumerate(_ranges(q_indptr, batch)):
        init = has_init is None or bool(has_init[b])
        s = state[int(slot_in[b])].float().clone() if init else torch.zeros(v_heads, vdim, kdim)
        for r in range(r0, r1):
            qv = q[r].float().view(k_heads, kdim)
            kv = k[r].float().view(k_heads, kdim)
            if l2norm:
                qv = qv * torch.rsqrt(qv.pow(2).sum(-1, keepdim=True) + 1e-6)
                kv = kv * torch.rsqrt(kv.pow(2).sum(-1, keepdim=True) + 1e-6)
            qv = (qv * scale).repeat_interleave(rep, 0)            # [v_heads, K]
            kv = kv.repeat_interleave(rep, 0)
            vv = v[r].float().view(v_heads, vdim)
            s = s * torch.exp(g[r].float())[:, None, None]
            u = (s * kv[:, None, :]).sum(-1)                       # [v_heads, V]
            dv = beta[r].float()[:, None] * (vv - u)
            s = s + dv[:, :, None] * kv[:, None, :]
            o[r] = (s * qv[:, None, :]).sum(-1).reshape(-1).to(q.dtype)
        if slot_out is not None:
            state[int(slot_out[b])] = s
    return o
