"""Row / pointwise ops: RMSNorm family, RoPE + q/k norm + KV-pool write, activations, embedding.

Each function runs the sm_100a kernel from csrc/misc.cu on CUDA tensors and a plain-PyTorch fp32 reference on
CPU tensors (the reference is also the oracle of the GPU numerics tests).
Reference counterparts: hibana/model/norm.py:14-71, hibana/model/rope.py:12, hibana/kernels/qk_norm_rope.py:16,
hibana/cache/kv_pool.py:120-132, hibana/kernels/flashnext_fused.py:624-660.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as nv

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_rmsnorm", [P, P, P, P, I, I, L, L, Fl, I, P])
nv.register("hb_gated_rmsnorm", [P, P, P, P, I, I, I, L, L, Fl, I, I, I, P])
nv.register("hb_gated_rmsnorm_quant", [P, P, P, I, I, I, L, L, Fl, I, I, I, P, P, P, I, P])
nv.register("hb_gdn_gates", [P, L, P, P, I, I, P, P, P])
nv.register("hb_rope_table", [P, P, I, I, P, P])
nv.register("hb_rope_use_table", [P], void=True)
nv.register("hb_rope_kv_write", [P, L, P, P, P, P, P, Fl, I, P, P, P, L, L, I, I, I, I, I, I, Fl, I, P])
nv.register("hb_act_mul", [P, P, P, L, I, L, I, P])
nv.register("hb_embedding", [P, P, P, I, I, L, P])
nv.register("hb_add", [P, P, P, L, P])

ACT_SILU_SPLIT, ACT_SILU_PAIRS, ACT_RELU2, ACT_SIGMOID_GATE = 0, 1, 2, 3


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *, residual: Optional[torch.Tensor] = None,
            gemma: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x [+ residual]) * w (gemma: (1 + w)). `residual` (contiguous) is updated in place."""
    rows, h = x.shape
    if nv.use_native(x):
        out = torch.empty(rows, h, dtype=x.dtype, device=x.device) if out is None else out
        nv.check(nv.lib().hb_rmsnorm(x.data_ptr(), nv.ptr(residual), weight.data_ptr(), out.data_ptr(), rows, h,
                                     x.stride(0), out.stride(0), eps, int(gemma), nv.stream()), "hb_rmsnorm")
        return out
    hsum = x
    if residual is not None:
        residual.copy_((x.float() + residual.float()).to(x.dtype))
        hsum = residual
    hf = hsum.float()
    w = weight.float() + 1.0 if gemma else weight.float()
    y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def gated_rmsnorm(x: torch.Tensor, z: Optional[torch.Tensor], weight: torch.Tensor, eps: float, group_size: int, *,
                  norm_first: bool = False, sigmoid_gate: bool = False, gemma: bool = False) -> torch.Tensor:
    """Grouped RMSNorm with a gate: rmsnorm_g(x * silu(z)) * w, or rmsnorm_g(x) * w * act(z) when norm_first."""
    rows, h = x.shape
    if nv.use_native(x):
        out = torch.empty(rows, h, dtype=x.dtype, device=x.device)
        nv.check(nv.lib().hb_gated_rmsnorm(x.data_ptr(), nv.ptr(z), weight.data_ptr(), out.data_ptr(), rows, h,
                                           group_size, x.stride(0), z.stride(0) if z is not None else 0, eps,
                                           int(norm_first), int(sigmoid_gate), int(gemma), nv.stream()),
                 "hb_gated_rmsnorm")
        return out
    xf = x.float()
    gate = None
    if z is not None:
        gate = torch.sigmoid(z.float()) if sigmoid_gate else F.silu(z.float())
    if gate is not None and not norm_first:
        xf = xf * gate
    g = xf.view(rows, h // group_size, group_size)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float() + 1.0 if gemma else weight.float()
    y = g.view(rows, h) * w
    if gate is not None and norm_first:
        y = y * gate
    return y.to(x.dtype)


def gated_rmsnorm_quant(x: torch.Tensor, z: Optional[torch.Tensor], weight: torch.Tensor, eps: float, group_size: int,
                        gscale: torch.Tensor, *, norm_first: bool = False, sigmoid_gate: bool = False,
                        gemma: bool = False):
    """`gated_rmsnorm` written as NVFP4 rows for the projection that follows (one kernel instead of norm + quantise)
    where the shape allows it (group size a multiple of 16 up to 1024, width a multiple of 64); otherwise the two
    steps. Returns an Nvfp4Tensor."""
    from . import nvfp4
    rows, h = x.shape
    ok = (nv.use_native(x) and group_size % 16 == 0 and group_size <= 1024 and h % 64 == 0 and x.stride(0) % 8 == 0
          and (z is None or z.stride(0) % 8 == 0))
    if not ok:
        return nvfp4.quantize(gated_rmsnorm(x, z, weight, eps, group_size, norm_first=norm_first,
                                            sigmoid_gate=sigmoid_gate, gemma=gemma), gscale)
    q, sf = nvfp4._alloc(rows, h, x.device)
    nv.check(nv.lib().hb_gated_rmsnorm_quant(x.data_ptr(), nv.ptr(z), weight.data_ptr(), rows, h, group_size,
                                             x.stride(0), z.stride(0) if z is not None else 0, eps, int(norm_first),
                                             int(sigmoid_gate), int(gemma), q.data_ptr(), sf.data_ptr(),
                                             gscale.data_ptr(), sf.shape[1], nv.stream()), "hb_gated_rmsnorm_quant")
    return nvfp4.Nvfp4Tensor(q, sf, gscale, rows, h)


def gdn_gates(ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Gated delta rule gates from the b | a projection ba [T, 2 * heads] (bf16): beta = sigmoid(b) and the log
    decay g = -exp(a_log) * softplus(a + dt_bias), both fp32 [T, heads], in one kernel."""
    rows, two = ba.shape
    heads = two // 2
    if nv.use_native(ba):
        beta = torch.empty(rows, heads, dtype=torch.float32, device=ba.device)
        g = torch.empty(rows, heads, dtype=torch.float32, device=ba.device)
        nv.check(nv.lib().hb_gdn_gates(ba.data_ptr(), ba.stride(0), a_log.data_ptr(), dt_bias.data_ptr(), rows, heads,
                                       beta.data_ptr(), g.data_ptr(), nv.stream()), "hb_gdn_gates")
        return beta, g
    f = ba.float()
    beta = torch.sigmoid(f[:, :heads]).contiguous()
    g = (-torch.exp(a_log.float()) * F.softplus(f[:, heads:] + dt_bias.float())).contiguous()
    return beta, g


def rope_inv_freq(rot_dim: int, theta: float, device=None) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))


def _norm_head(t: torch.Tensor, w: Optional[torch.Tensor], eps: float, gemma: bool) -> torch.Tensor:
    if w is None:
        return t
    ww = w.float() + 1.0 if gemma else w.float()
    return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * ww).to(torch.bfloat16).float()


def _rope_ref(t: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, rot: int) -> torch.Tensor:
    """NeoX rotary on the first `rot` dims of t [T, H, D] (fp32)."""
    if rot == 0:
        return t
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = t[..., : rot // 2], t[..., rot // 2: rot]
    out = t.clone()
    out[..., : rot // 2] = a * cos - b * sin
    out[..., rot // 2: rot] = b * cos + a * sin
    return out


ROPE_TABLE_MIN_ROWS = 256     # below this a layer's own sincos is cheaper than one more launch per forward


def rope_table(ctx, inv_freq: torch.Tensor, rot: int) -> Optional[torch.Tensor]:
    """(cos, sin) of every row's rotary angles, fp32 [T, rot / 2, 2], computed once per forward (cached in
    `ctx.extras`) and read by every layer's `rope_kv_write`: a prefill chunk otherwise evaluates the same sincos in
    each of its layers. None for small row counts and on the CPU path."""
    pos = ctx.positions
    if pos is None or not pos.is_cuda or pos.shape[0] < ROPE_TABLE_MIN_ROWS or rot < 2:
        return None
    key = ("rope_table", rot)
    tab = ctx.extras.get(key)
    if tab is None:
        tab = torch.empty(pos.shape[0], rot // 2, 2, dtype=torch.float32, device=pos.device)
        nv.check(nv.lib().hb_rope_table(pos.data_ptr(), inv_freq.data_ptr(), pos.shape[0], rot // 2, tab.data_ptr(),
                                        nv.stream()), "hb_rope_table")
        ctx.extras[key] = tab
    return tab


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor], inv_freq: torch.Tensor,
                  k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], hq: int, hkv: int, d: int, *,
                  rot: Optional[int] = None, q_norm: Optional[torch.Tensor] = None,
                  k_norm: Optional[torch.Tensor] = None, eps: float = 1e-6, gemma_norm: bool = False,
                  kv_scale: float = 1.0, q_gate: bool = False, table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Splits a fused qkv row, applies per-head q/k RMSNorm and NeoX RoPE, writes K/V rows into the pools.
    `table` (`rope_table`): the rows' (cos, sin) angles computed once per forward instead of in every layer.

    qkv [T, Hq*D(*2 with q_gate) + 2*Hkv*D] bf16; positions / slots int32 [T]; pools [slots, Hkv, D] (bf16 or
    float8_e4m3fn scaled by 1/kv_scale). Returns q [T, Hq, D] bf16. `slots=None` skips the pool write.
    """
    t = qkv.shape[0]
    rot = d if rot is None else rot
    qw = hq * d * (2 if q_gate else 1)
    k_sf = getattr(k_pool, "sf", None) if k_pool is not None else None      # NVFP4 pool: scale rows ride along
    if nv.use_native(qkv):
        q_out = torch.empty(t, hq, d, dtype=torch.bfloat16, device=qkv.device)
        fp8 = k_pool is not None and k_pool.dtype != torch.bfloat16
        if k_sf is not None:
            fp8 = 2
            nv.register("hb_kv_fp4_scales", [nv.P, nv.P, nv.L, nv.L], void=True)
            nv.lib().hb_kv_fp4_scales(k_sf.data_ptr(), v_pool.sf.data_ptr(), k_sf.stride(0), k_sf.stride(1))
        if table is not None:
            nv.lib().hb_rope_use_table(table.data_ptr())
        nv.check(nv.lib().hb_rope_kv_write(
            qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), nv.ptr(slots), inv_freq.data_ptr(), nv.ptr(q_norm),
            nv.ptr(k_norm), eps, int(gemma_norm), q_out.data_ptr(), nv.ptr(k_pool), nv.ptr(v_pool),
            k_pool.stride(0) if k_pool is not None else 0, k_pool.stride(1) if k_pool is not None else 0, t, hq,
            hkv, d, rot, int(fp8), 1.0 / kv_scale, int(q_gate), nv.stream()), "hb_rope_kv_write")
        return q_out
    x = qkv.float()
    if q_gate:
        q = x[:, :qw].view(t, hq, 2 * d)[..., :d]
    else:
        q = x[:, :qw].view(t, hq, d)
    k = x[:, qw: qw + hkv * d].view(t, hkv, d)
    v = x[:, qw + hkv * d:].view(t, hkv, d)
    q = _rope_ref(_norm_head(q, q_norm, eps, gemma_norm), positions, inv_freq, rot)
    k = _rope_ref(_norm_head(k, k_norm, eps, gemma_norm), positions, inv_freq, rot)
    if slots is not None and k_pool is not None:
        idx = slots.long()
        if k_sf is not None:
            from . import nvfp4
            for pool, x_ in ((k_pool, k), (v_pool, v)):
                rows = x_.to(torch.bfloat16).float().reshape(t * hkv, d)
                packed, sfb = nvfp4.quantize_ref(rows, kv_scale)
                pool[idx] = packed.view(t, hkv, d // 2)
                pool.sf[idx] = sfb.view(t, hkv, d // 16)
        elif k_pool.dtype == torch.bfloat16:
            k_pool[idx] = k.to(torch.bfloat16)
            v_pool[idx] = v.to(torch.bfloat16)
        else:
            k_pool[idx] = (k / kv_scale).clamp(-448, 448).to(k_pool.dtype)
            v_pool[idx] = (v / kv_scale).clamp(-448, 448).to(v_pool.dtype)
    return q.to(torch.bfloat16)


def act_mul(x: torch.Tensor, mode: int = ACT_SILU_SPLIT, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate)*up on [T, 2I] (split halves or interleaved pairs), relu(x)^2, or x * sigmoid(gate)."""
    rows = x.shape[0]
    inter = x.shape[1] // 2 if mode in (ACT_SILU_SPLIT, ACT_SILU_PAIRS) else x.shape[1]
    if nv.use_native(x):
        out = torch.empty(rows, inter, dtype=x.dtype, device=x.device)
        nv.check(nv.lib().hb_act_mul(x.data_ptr(), nv.ptr(gate), out.data_ptr(), rows, inter, x.stride(0), mode,
                                     nv.stream()), "hb_act_mul")
        return out
    xf = x.float()
    if mode == ACT_SILU_SPLIT:
        y = F.silu(xf[:, :inter]) * xf[:, inter:]
    elif mode == ACT_SILU_PAIRS:
        y = F.silu(xf[:, 0::2]) * xf[:, 1::2]
    elif mode == ACT_RELU2:
        y = torch.relu(xf) ** 2
    else:
        y = xf * torch.sigmoid(gate.float())
    return y.to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if nv.use_native(ids, table):
        out = torch.empty(ids.shape[0], table.shape[1], dtype=table.dtype, device=table.device)
        nv.check(nv.lib().hb_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.shape[0],
                                       table.shape[1], table.shape[0], nv.stream()), "hb_embedding")
        return out
    return table[ids.clamp(0, table.shape[0] - 1)]


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if nv.use_native(a, b):
        out = torch.empty_like(a)
        nv.check(nv.lib().hb_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), nv.stream()), "hb_add")
        return out
    return (a.float() + b.float()).to(a.dtype)
