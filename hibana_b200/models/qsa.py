"""Sparse attention indexer ("QSA"): choose, per query row, which KV tokens full attention may look at.

Every `ratio` consecutive tokens form a group with one compressed index key (mean of the tokens' raw index keys,
Gemma RMSNorm, RoPE at the group's first position). A query row at position i scores the (i + 1) // ratio complete
groups with sum_h relu(q_h . k) / sqrt(D), keeps the best budget // ratio, and adds the tail of its own incomplete
group. The result is a per-row KV slot list that the paged attention kernels consume as that row's block table
(non-causal: the list already encodes causality). With no more than budget // ratio groups everything is kept, i.e.
the result equals dense causal attention. Kernels: csrc/qsa.cu; top-k by torch.topk on the device.
Reference: hibana/model/flashnext/reference.py:29-64 (rule and torch oracle), hibana/model/flashnext/indexer.py.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as nv
from ..ops import attention, basic

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_qsa_compress", [P, P, P, L, P, P, P, I, I, I, P, Fl, P, I, P])
nv.register("hb_qsa_score", [P, I, I, P, P, L, P, P, I, I, P, P])
nv.register("hb_qsa_expand", [P, P, I, I, P, L, P, P, I, P, L, P, P])

QD = 128


def _rope(x: torch.Tensor, pos: torch.Tensor, rot: int, inv_freq: torch.Tensor) -> torch.Tensor:
    ang = pos.float()[:, None] * inv_freq[None, :rot // 2].float()
    c, s = ang.cos(), ang.sin()
    a, b = x[..., :rot // 2].float(), x[..., rot // 2:rot].float()
    shape = (-1,) + (1,) * (x.dim() - 2) + (rot // 2,)
    c, s = c.view(shape), s.view(shape)
    return torch.cat([a * c - b * s, b * c + a * s, x[..., rot:].float()], dim=-1)


def compress_ref(raw_k, kv_indices, seq_rows, first, count, ratio, norm_w, eps, inv_freq, rot, ckey) -> None:
    for b in range(len(first)):
        idx = kv_indices[int(seq_rows[b]) if seq_rows is not None else b]
        for g in range(int(first[b]), int(first[b]) + int(count[b])):
            sl = idx[g * ratio:(g + 1) * ratio].long()
            m = raw_k[sl].float().mean(0)
            m = (m * torch.rsqrt(m.pow(2).mean() + eps) * (1 + norm_w.float())).to(torch.bfloat16).float()
            ckey[sl[0]] = _rope(m[None, :], torch.tensor([g * ratio]), rot, inv_freq)[0].to(ckey.dtype)


def select_ref(q, ckey, kv_indices, row_seq, row_pos, ratio, budget):
    """Per row: list of KV slots (chosen groups' tokens + tail)."""
    out = []
    for r in range(q.shape[0]):
        idx = kv_indices[int(row_seq[r])]
        pos = int(row_pos[r])
        vis = (pos + 1) // ratio
        slots: list[int] = []
        if vis:
            keys = ckey[idx[torch.arange(vis) * ratio].long()].float()
            sc = torch.relu(torch.einsum("hd,gd->gh", q[r].float(), keys)).sum(-1) / QD ** 0.5
            top = torch.topk(sc, min(budget // ratio, vis)).indices.tolist()
            for g in top:
                slots += idx[g * ratio:(g + 1) * ratio].tolist()
        slots += idx[vis * ratio:pos + 1].tolist()
        out.append(slots)
    return out


class QsaIndexer:
    def __init__(self, ratio: int = 4, budget: int = 2048, heads: int = 4, rot: int = 64, eps: float = 1e-6,
                 theta: float = 1e6, device="cpu"):
        self.ratio, self.budget, self.heads, self.rot, self.eps = ratio, budget, heads, rot, eps
        self.device = torch.device(device)
        self.inv_freq = basic.rope_inv_freq(rot, theta, device=self.device)
        self.norm_w = torch.zeros(QD, dtype=torch.bfloat16, device=self.device)

    def compress(self, raw_k: torch.Tensor, ckey: torch.Tensor, kv_indices: torch.Tensor,
                 seq_rows: Optional[torch.Tensor], first: torch.Tensor, count: torch.Tensor,
                 max_total: Optional[int] = None) -> None:
        """Writes the compressed keys of groups [first[b], first[b] + count[b]) of every sequence b into `ckey`
        (row = slot of the group's first token). raw_k / ckey: [slots, 128] bf16 pools. `max_total`: an upper bound
        of sum(count) known on the host; with it the call needs no device-to-host read (CUDA graphs): the grid
        covers the bound and CTAs beyond the real total return."""
        if not nv.use_native(raw_k):
            compress_ref(raw_k, kv_indices, seq_rows, first, count, self.ratio, self.norm_w, self.eps, self.inv_freq,
                         self.rot, ckey)
            return
        indptr = torch.zeros(first.numel() + 1, dtype=torch.int32, device=raw_k.device)
        indptr[1:] = count.cumsum(0)
        total = int(indptr[-1]) if max_total is None else int(max_total)
        if total <= 0:
            return
        nv.check(nv.lib().hb_qsa_compress(raw_k.data_ptr(), ckey.data_ptr(), kv_indices.data_ptr(),
                                          kv_indices.stride(0), nv.ptr(seq_rows), indptr.data_ptr(),
                                          first.data_ptr(), first.numel(), total, self.ratio, self.norm_w.data_ptr(),
                                          self.eps, self.inv_freq.data_ptr(), self.rot, nv.stream()), "hb_qsa_compress")

    def select(self, q: torch.Tensor, ckey: torch.Tensor, kv_indices: torch.Tensor, row_seq: torch.Tensor,
               row_pos: torch.Tensor, max_pos: int) -> tuple[torch.Tensor, torch.Tensor]:
        """q [rows, heads, 128] (normed, rotated index queries). Returns (sel int32 [rows, budget + ratio], sel_len
        int32 [rows]): the KV slots every row attends to."""
        rows = q.shape[0]
        width_tokens = self.budget + self.ratio
        if not nv.use_native(q):
            lists = select_ref(q, ckey, kv_indices, row_seq, row_pos, self.ratio, self.budget)
            sel = torch.zeros(rows, width_tokens, dtype=torch.int32)
            for r, ls in enumerate(lists):
                sel[r, :len(ls)] = torch.tensor(ls, dtype=torch.int32)
            return sel, torch.tensor([len(ls) for ls in lists], dtype=torch.int32)
        dev = q.device
        max_groups = max((max_pos + 1) // self.ratio, 1)
        scores = torch.empty(rows, max_groups, dtype=torch.float32, device=dev)
        nv.check(nv.lib().hb_qsa_score(q.data_ptr(), rows, self.heads, ckey.data_ptr(), kv_indices.data_ptr(),
                                       kv_indices.stride(0), row_seq.data_ptr(), row_pos.data_ptr(), self.ratio,
                                       max_groups, scores.data_ptr(), nv.stream()), "hb_qsa_score")
        width = min(self.budget // self.ratio, max_groups)
        vals, chosen = torch.topk(scores, width, dim=-1)
        sel = torch.zeros(rows, width_tokens, dtype=torch.int32, device=dev)
        sel_len = torch.empty(rows, dtype=torch.int32, device=dev)
        nv.check(nv.lib().hb_qsa_expand(chosen.data_ptr(), vals.data_ptr(), rows, width, kv_indices.data_ptr(),
                                        kv_indices.stride(0), row_seq.data_ptr(), row_pos.data_ptr(), self.ratio,
                                        sel.data_ptr(), sel.stride(0), sel_len.data_ptr(), nv.stream()), "hb_qsa_expand")
        return sel, sel_len

    @staticmethod
    def sparse_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, sel: torch.Tensor,
                         sel_len: torch.Tensor, scale: Optional[float] = None, kv_scale: float = 1.0) -> torch.Tensor:
        """Full attention of every query row over its own slot list (each row is its own one-row 'sequence')."""
        return attention.paged_attention(q, k_pool, v_pool, sel, sel_len, causal=False, scale=scale,
                                         kv_scale=kv_scale,
                                         splits=attention.choose_splits(q.shape[0], k_pool.shape[1], sel.shape[1]))
