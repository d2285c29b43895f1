"""Paged GQA attention over the token-granular KV pool (decode, speculative verify, chunked prefill).

`paged_attention` is the single entry: query rows of a ragged batch attend to their sequence's context through
the block table. Kernels: csrc/attn_prefill.cu (tcgen05 prefill), csrc/attn_decode.cu (tensor-core flash-decoding,
up to 16 query rows per kv head), csrc/attn.cu (general split-KV + LSE merge; fp8 KV, head dim 256 prefill). The plain-PyTorch reference below is the CPU path
and the GPU tests' oracle. Reference counterparts: hibana/kernels/ops.py:131-161 (ragged prefill),
hibana/model/attention.py:69-126, hibana/kernels/csrc/verify_attn.cu.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native as nv
from .. import config as cfgmod
from . import nvfp4

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_attn_paged", [P, P, P, L, L, P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, Fl, I, Fl, I, P])

nv.register("hb_attn_merge", [P, P, P, L, I, I, P])
nv.register("hb_attn_fp4_scales", [P, P, L, L], void=True)
nv.register("hb_attn_merge_quant", [P, P, L, I, I, I, P, P, P, I, P])
nv.register("hb_attn_decode", [P, P, P, L, L, P, L, P, P, P, P, P, P, I, I, I, I, I, I, Fl, I, L, P, P])

nv.register("hb_attn_decode_fuse", [P, P, P, P, I], void=True)
nv.register("hb_attn_decode_tc", [P, P, P, L, L, P, L, P, P, P, P, P, P, I, I, I, I, I, I, Fl, I, L, P, P])
nv.register("hb_attn_decode_tc_profile", [P], void=True)
nv.register("hb_attn_prefill_profile", [P], void=True)
nv.register("hb_attn_decode_profile", [P], void=True)
nv.register("hb_attn_prefill", [P, P, P, L, L, P, L, P, P, P, P, I, I, I, I, I, Fl, I, L, P, P])

from ..hardware.b200 import NUM_SMS  # noqa: E402


DECODE_CTAS_PER_SM = 2      # csrc/attn_decode.cu: 64-thread CTAs with ~100 KB of rings, two share an SM


def choose_splits(batch: int, hkv: int, max_ctx: int, row_chunks: int = 1, slots: int = 0) -> int:
    """KV splits that fill whole waves of the resident CTA slots (the decode kernel streams from every resident
    CTA at once, so a last wave that is a third full costs a whole wave); a split never gets fewer than 256 keys."""
    if cfgmod.current().stable_numerics:
        # row-count invariant: one pass over the keys in fixed tiles from position 0, so a token's attention sums
        # in the same order whether it is the only new row of its sequence or one of several verified rows
        return 1
    slots = slots or NUM_SMS * max(1, cfgmod.current().attn_ctas_per_sm)
    ctas = max(1, batch * hkv * row_chunks)
    cap = int(max(1, min(max_ctx // 256, 64)))
    best, best_eff = 1, 0.0
    for s in range(1, cap + 1):
        n = ctas * s
        eff = n / (-(-n // slots) * slots)
        if eff > best_eff + 0.02:     # prefer fewer splits unless the wave efficiency clearly improves
            best, best_eff = s, eff
    return best


class AttnWorkspace:
    """Split-KV partial buffers, allocated once (stable addresses for CUDA graphs)."""

    def __init__(self, rows: int, hq: int, d: int, splits: int, device: torch.device):
        self.rows, self.splits = rows, splits
        self.part_o = torch.empty(rows, hq, splits, d, dtype=torch.float32, device=device)
        self.part_lse = torch.empty(rows, hq, splits, dtype=torch.float32, device=device)
        # arrivals per (sequence, kv head) of the fused split merge: zero between launches (the kernel re-arms it)
        self.counter = torch.zeros(rows * hq, dtype=torch.int32, device=device)


def paged_attention_ref(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, kv_indices: torch.Tensor,
                        ctx_len: torch.Tensor, q_indptr: Optional[torch.Tensor], scale: float, kv_scale: float = 1.0,
                        causal: bool = True) -> torch.Tensor:
    t, hq, d = q.shape
    hkv = k_pool.shape[1]
    g = hq // hkv
    out = torch.zeros(t, hq, d, dtype=torch.float32, device=q.device)
    b = ctx_len.shape[0]
    for i in range(b):
        r0 = int(q_indptr[i]) if q_indptr is not None else i
        r1 = int(q_indptr[i + 1]) if q_indptr is not None else i + 1
        rows = r1 - r0
        ctx = int(ctx_len[i])
        if rows == 0 or ctx == 0:
            continue
        idx = kv_indices[i, :ctx].long()
        if getattr(k_pool, "sf", None) is not None:     # NVFP4 pool: packed values + block scales
            from ..cache.kv_pool import dequant_rows
            k = dequant_rows(k_pool[idx], k_pool.sf[idx], kv_scale)
            v = dequant_rows(v_pool[idx], v_pool.sf[idx], kv_scale)
        else:
            k = k_pool[idx].float() * kv_scale     # [ctx, hkv, d]
            v = v_pool[idx].float() * kv_scale
        qq = q[r0:r1].float().view(rows, hkv, g, d)
        s = torch.einsum("rhgd,chd->rhgc", qq, k) * scale
        if causal:
            pos = torch.arange(ctx, device=q.device)[None, :]
            lim = (ctx - rows + torch.arange(rows, device=q.device))[:, None]
            s = s.masked_fill((pos > lim)[:, None, None, :], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[r0:r1] = torch.einsum("rhgc,chd->rhgd", p, v).reshape(rows, hq, d)
    return out.to(q.dtype)


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, kv_indices: torch.Tensor,
                    ctx_len: torch.Tensor, *, q_indptr: Optional[torch.Tensor] = None, max_rows: int = 1,
                    seq_rows: Optional[torch.Tensor] = None,
                    scale: Optional[float] = None, kv_scale: float = 1.0, causal: bool = True, splits: int = 1,
                    workspace: Optional[AttnWorkspace] = None, out: Optional[torch.Tensor] = None,
                    quant_scale: Optional[torch.Tensor] = None):
    """q [T, Hq, D] bf16; pools [slots, Hkv, D]; kv_indices [B, max_ctx] int32; ctx_len [B] int32.

    Row r of sequence b (rows q_indptr[b]..q_indptr[b+1], or exactly one row when q_indptr is None) sees keys
    [0, ctx_len[b] - rows_b + r + 1) when causal. `max_rows` bounds rows per sequence (host value).
    `seq_rows` int32 [B] selects each sequence's row of kv_indices (identity when None).
    `quant_scale` (fp32 scalar tensor): return the rows [T, Hq * D] as an Nvfp4Tensor quantised with that static
    scale (the activation operand of the output projection); on the decode kernel this and the split merge happen
    inside the attention kernel, elsewhere a quantisation pass follows.
    """
    t, hq, d = q.shape
    hkv = k_pool.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if not nv.use_native(q, k_pool):
        idx = kv_indices if seq_rows is None else kv_indices[seq_rows.long()]
        res = paged_attention_ref(q, k_pool, v_pool, idx, ctx_len, q_indptr, scale, kv_scale, causal)
        if out is not None:
            out.copy_(res)
            res = out
        return res if quant_scale is None else nvfp4.quantize(res.reshape(t, hq * d), quant_scale)
    b = ctx_len.shape[0]
    if splits > 1 and (workspace is None or workspace.rows < t or workspace.splits != splits):
        workspace = AttnWorkspace(t, hq, d, splits, q.device)
    fp4 = getattr(k_pool, "sf", None) is not None
    fp8 = k_pool.dtype != torch.bfloat16
    cfg = cfgmod.current()
    if not fp8 and max_rows * (hq // hkv) <= 16 and d in (64, 128, 256):
        st = nv.device_state(q.device)
        tc = d == 128 and cfg.decode_attn == "tc"
        fuse = cfg.fuse_epilogues and not tc and (cfg.fuse_attn_tail or splits == 1)
        xq = None
        if fuse:
            qb = sfb = None
            if quant_scale is not None:
                qb, sfb = _quant_bufs(t, hq * d, q.device)
                xq = nvfp4.Nvfp4Tensor(qb, sfb, quant_scale, t, hq * d)
            nv.lib().hb_attn_decode_fuse(workspace.counter.data_ptr() if splits > 1 else None, nv.ptr(qb), nv.ptr(sfb),
                                         nv.ptr(quant_scale), sfb.shape[1] if sfb is not None else 0)
        if xq is None:
            out = torch.empty_like(q) if out is None else out
        # decode_attn = "tc" selects the persistent tcgen05 kernel (head dim 128; csrc/attn_decode_tc.cu). It
        # matches the mma.sync kernel in isolation (123 vs 122 us at 64 x 2304 keys) but not yet inside the 27B
        # decode step (18.8 vs 15.8 ms per step), so the mma.sync kernel stays the default.
        args = (q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.stride(0), k_pool.stride(1),
                kv_indices.data_ptr(), kv_indices.stride(0), nv.ptr(seq_rows), ctx_len.data_ptr(), nv.ptr(q_indptr),
                nv.ptr(out), workspace.part_o.data_ptr() if splits > 1 else None,
                workspace.part_lse.data_ptr() if splits > 1 else None, b, max_rows, hq, hkv, d, splits, scale,
                int(causal), k_pool.shape[0], st.status.data_ptr())
        fn = nv.lib().hb_attn_decode_tc if tc else nv.lib().hb_attn_decode
        nv.check(fn(*args, nv.stream()), "hb_attn_decode")
        if xq is not None:
            return xq
        if splits > 1 and not fuse:
            if quant_scale is not None and cfg.fuse_epilogues:
                # the merge kernel writes the NVFP4 rows itself: no separate quantisation pass
                qb, sfb = _quant_bufs(t, hq * d, q.device)
                nv.check(nv.lib().hb_attn_merge_quant(workspace.part_o.data_ptr(), workspace.part_lse.data_ptr(), t,
                                                      hq, splits, d, qb.data_ptr(), sfb.data_ptr(),
                                                      quant_scale.data_ptr(), sfb.shape[1], nv.stream()),
                         "hb_attn_merge_quant")
                return nvfp4.Nvfp4Tensor(qb, sfb, quant_scale, t, hq * d)
            nv.check(nv.lib().hb_attn_merge(workspace.part_o.data_ptr(), workspace.part_lse.data_ptr(),
                                            out.data_ptr(), t * hq, splits, d, nv.stream()), "hb_attn_merge")
        return out if quant_scale is None else nvfp4.quantize(out.view(t, hq * d), quant_scale)
    out = torch.empty_like(q) if out is None else out
    res = _paged_general(q, k_pool, v_pool, kv_indices, ctx_len, q_indptr, max_rows, seq_rows, scale, kv_scale, causal,
                         splits, workspace, out, cfg, fp8, b, t, hq, hkv, d)
    return res if quant_scale is None else nvfp4.quantize(res.view(t, hq * d), quant_scale)


_QUANT_BUFS: dict = {}


def _quant_bufs(rows: int, k: int, device):
    """Persistent NVFP4 output buffers per shape (stable addresses for captured graphs); padding scales zeroed once."""
    key = (device, rows, k)
    bufs = _QUANT_BUFS.get(key)
    if bufs is None:
        qb, sfb = nvfp4._alloc(rows, k, device)
        sfb.zero_()
        bufs = _QUANT_BUFS[key] = (qb, sfb)
    return bufs


def _paged_general(q, k_pool, v_pool, kv_indices, ctx_len, q_indptr, max_rows, seq_rows, scale, kv_scale, causal,
                   splits, workspace, out, cfg, fp8, b, t, hq, hkv, d):
    if getattr(k_pool, "sf", None) is not None:
        fp8 = 2       # NVFP4 pool: the split-KV kernel dequantises rows as it loads them
        nv.lib().hb_attn_fp4_scales(k_pool.sf.data_ptr(), v_pool.sf.data_ptr(), k_pool.sf.stride(0), k_pool.sf.stride(1))
    if not fp8 and d in (64, 128, 256) and q_indptr is not None and cfg.prefill_attn == "tc":
        st = nv.device_state(q.device)
        nv.check(nv.lib().hb_attn_prefill(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.stride(0), k_pool.stride(1), kv_indices.data_ptr(),
            kv_indices.stride(0), nv.ptr(seq_rows), ctx_len.data_ptr(), q_indptr.data_ptr(), out.data_ptr(), b,
            max_rows, hq, hkv, d, scale, int(causal), k_pool.shape[0], st.status.data_ptr(), nv.stream()),
                 "hb_attn_prefill")
        return out
    nv.check(nv.lib().hb_attn_paged(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.stride(0), k_pool.stride(1), kv_indices.data_ptr(),
        kv_indices.stride(0), nv.ptr(seq_rows), ctx_len.data_ptr(), nv.ptr(q_indptr), out.data_ptr(),
        workspace.part_o.data_ptr() if splits > 1 else None, workspace.part_lse.data_ptr() if splits > 1 else None,
        b, t, max_rows, hq, hkv, d, splits, scale, int(fp8), kv_scale, int(causal), nv.stream()), "hb_attn_paged",
             launches=2 if splits > 1 else 1)
    return out


TC_PROFILE_FIELDS = ("producer_wait", "tiles_tma", "tiles_gather", "issuer_wait_full", "issuer_wait_p",
                     "softmax_wait_s", "softmax_wait_pv", "epilogue", "softmax_total", "raises", "tiles", "ctas")


class DecodeTcProfile:
    """Role counters of the tcgen05 decode kernel (csrc/attn_decode_tc.cu), accumulated while the object lives."""

    def __init__(self, device):
        self.buf = torch.zeros(len(TC_PROFILE_FIELDS), dtype=torch.int64, device=device)
        nv.lib().hb_attn_decode_tc_profile(self.buf.data_ptr())

    def read(self) -> dict:
        torch.cuda.synchronize(self.buf.device)
        c = dict(zip(TC_PROFILE_FIELDS, self.buf.tolist()))
        tiles, ctas = max(c["tiles"], 1), max(c["ctas"], 1)
        out = {k: round(c[k] / tiles) for k in ("producer_wait", "issuer_wait_full", "issuer_wait_p",
                                                "softmax_wait_s", "softmax_wait_pv")}
        out.update(epilogue_per_cta=round(c["epilogue"] / ctas), total_per_cta=round(c["softmax_total"] / ctas),
                   tiles_per_cta=round(tiles / ctas, 1), raises_per_tile=round(c["raises"] / tiles, 3),
                   gather_share=round(c["tiles_gather"] / max(c["tiles_gather"] + c["tiles_tma"], 1), 3))
        return out

    def close(self) -> None:
        nv.lib().hb_attn_decode_tc_profile(None)
