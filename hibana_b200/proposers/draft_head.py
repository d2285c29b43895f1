"""Draft heads: how a drafter turns hidden rows into token choices.

Every speculator ends in a vocabulary projection. The default is the target's own head (`TargetHead`). A
`ShortlistHead` reads fewer bytes per draft step: a subset of the head's rows (a reduced draft vocabulary), a 3-bit
copy of them (the dequant-fused tcgen05 GEMM of ops/w3gemm.py), or both, with the leading candidates rescored
against the target's own bf16 rows so that the pick is the full head's whenever its argmax is on the shortlist.
A `VocabParallelHead` serves a vocabulary-parallel lm_head under tensor parallelism: each rank scores only its rows
and the ranks agree through two small gathers (rows x ranks x r values and ids) instead of the whole logits.
The target still verifies with its own head, so under exact acceptance a cheaper draft head changes how many drafts
are accepted, never what is emitted. Reference: hibana/proposers/draft_head.py:28-340.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..ops import gemm

FORMATS = ("bf16", "w3")
DEFAULT_RESCORE = {"w3": 8}


def confidence(logits: torch.Tensor) -> torch.Tensor:
    """[..., V] logits -> fp32 [..., 2]: the top-1 softmax probability and its margin over the top-2."""
    top = torch.softmax(logits.float(), dim=-1).topk(2, dim=-1).values
    return torch.stack([top[..., 0], top[..., 0] - top[..., 1]], dim=-1)


class TargetHead:
    """The target's vocabulary projection as a draft head."""
    rows_changed = False

    def __init__(self, logits_fn: Callable[[torch.Tensor], torch.Tensor]):
        self.logits_fn = logits_fn

    @property
    def bytes(self) -> int:
        return 0          # already resident

    def logits(self, x: torch.Tensor) -> torch.Tensor:
        return self.logits_fn(x)

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        return self.logits_fn(x).argmax(-1)

    def argmax_confidence(self, x: torch.Tensor):
        lg = self.logits_fn(x)
        return lg.argmax(-1), confidence(lg)

    def candidates(self, x: torch.Tensor, r: int):
        """(global ids int64 [..., r], fp32 logits [..., r]) of the r best tokens, descending."""
        v, i = self.logits_fn(x).topk(r, dim=-1)
        return i, v.float()


def _pad_rows(ids: torch.Tensor, multiple: int) -> torch.Tensor:
    pad = (-ids.numel()) % multiple
    return torch.cat((ids, ids[-1:].expand(pad))) if pad else ids


class ShortlistHead:
    """Rows `ids` of a bf16 lm_head [V, H] (all rows when `ids` is None), as they are (`fmt="bf16"`) or as a 3-bit
    copy (`"w3"`); with `rescore` > 1 the copy's logits only nominate that many candidates and the target head's
    own rows choose among them."""
    rows_changed = True

    def __init__(self, lm_head: torch.Tensor, ids: Optional[torch.Tensor] = None, fmt: str = "bf16", rescore: int = 0):
        if fmt not in FORMATS:
            raise ValueError(f"draft head format must be one of {FORMATS}, not {fmt!r}")
        if lm_head.dim() != 2:
            raise ValueError("a shortlist draft head reads rows of a [vocab, hidden] lm_head")
        self.fmt, self.source = fmt, lm_head
        self.ids = None if ids is None else ids.to(lm_head.device, torch.int64).unique(sorted=True)
        self.real_rows = lm_head.shape[0] if self.ids is None else self.ids.numel()
        if fmt == "w3" and self.ids is not None:
            self.ids = _pad_rows(self.ids, 128)           # whole 128-row tiles; padding repeats the last id
        rows = lm_head if self.ids is None else lm_head[self.ids].contiguous()
        self.w3 = None
        if fmt == "w3":
            from ..ops.w3gemm import W3Linear
            if self.ids is None and rows.shape[0] % 128:
                pad = (-rows.shape[0]) % 128
                rows = torch.cat((rows, rows[-1:].expand(pad, -1)))
            self.w3 = W3Linear.from_weight(rows.float(), lm_head.device, name="draft_head")
            self.rows = None
        else:
            self.rows = rows
        self.rescore = rescore if fmt != "bf16" and rescore > 1 else 0

    @property
    def bytes(self) -> int:
        """Bytes this head adds beside the target's lm_head."""
        if self.w3 is not None:
            return self.w3.nbytes()
        return 0 if self.ids is None else self.rows.numel() * 2

    def _logits(self, flat: torch.Tensor) -> torch.Tensor:
        if self.w3 is not None:
            lg = self.w3(flat.contiguous()).float()
        else:
            lg = gemm.linear_bf16(flat.contiguous(), self.rows, epilogue=gemm.EPI_STORE_F32)
        return lg[:, :self.real_rows] if lg.shape[1] != self.real_rows and self.ids is None else lg

    def _global(self, local: torch.Tensor) -> torch.Tensor:
        return local if self.ids is None else self.ids[local]

    def _rescored(self, flat: torch.Tensor, lg: torch.Tensor, r: int):
        """Top-r of the copy's logits re-ordered by the source head's own rows: (global ids [M, r], logits [M, r])."""
        cand = self._global(lg.topk(r, dim=-1).indices)
        rows = self.source[cand].float()                                    # [M, r, H]
        exact = torch.bmm(rows, flat.float().unsqueeze(-1)).squeeze(-1)
        order = exact.argsort(dim=-1, descending=True)
        return cand.gather(-1, order), exact.gather(-1, order)

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.reshape(-1, x.shape[-1])
        lg = self._logits(flat)
        if self.rescore:
            ids, _ = self._rescored(flat, lg, self.rescore)
            return ids[:, 0].view(x.shape[:-1])
        return self._global(lg.argmax(-1)).view(x.shape[:-1])

    def argmax_confidence(self, x: torch.Tensor):
        flat = x.reshape(-1, x.shape[-1])
        lg = self._logits(flat)
        return self.argmax(x), confidence(lg).view(*x.shape[:-1], 2)

    def candidates(self, x: torch.Tensor, r: int):
        flat = x.reshape(-1, x.shape[-1])
        lg = self._logits(flat)
        if self.rescore:
            ids, v = self._rescored(flat, lg, max(self.rescore, r))
            ids, v = ids[:, :r], v[:, :r]
        else:
            v, local = lg.topk(r, dim=-1)
            ids = self._global(local)
        return ids.view(*x.shape[:-1], r), v.float().view(*x.shape[:-1], r)


class VocabParallelHead:
    """Draft head over a vocabulary-parallel lm_head shard [V / tp, H]: every rank proposes its r best (values and
    global ids), one gather of rows x tp x r pairs brings them together, and every rank takes the same best of
    those. With `rescore` the nominated candidates are re-scored by the rank that holds their bf16 row and summed
    over ranks (exactly one rank contributes to each candidate)."""
    rows_changed = True

    def __init__(self, shard: torch.Tensor, comm, rank: int, fmt: str = "bf16", rescore: int = 0):
        if fmt not in FORMATS:
            raise ValueError(f"draft head format must be one of {FORMATS}, not {fmt!r}")
        self.shard, self.comm, self.fmt = shard, comm, fmt
        self.local = shard.shape[0]
        self.offset = rank * self.local
        self.w3 = None
        if fmt == "w3":
            from ..ops.w3gemm import W3Linear
            rows = shard
            if rows.shape[0] % 128:
                rows = torch.cat((rows, rows[-1:].expand((-rows.shape[0]) % 128, -1)))
            self.w3 = W3Linear.from_weight(rows.float(), shard.device, name="draft_head_shard")
        self.rescore = rescore if fmt != "bf16" and rescore > 1 else 0

    @property
    def bytes(self) -> int:
        return self.w3.nbytes() if self.w3 is not None else 0

    def _logits(self, flat: torch.Tensor) -> torch.Tensor:
        if self.w3 is not None:
            return self.w3(flat.contiguous()).float()[:, :self.local]
        return gemm.linear_bf16(flat.contiguous(), self.shard, epilogue=gemm.EPI_STORE_F32)

    def candidates(self, x: torch.Tensor, r: int):
        flat = x.reshape(-1, x.shape[-1])
        width = max(self.rescore, r)
        v, local = self._logits(flat).topk(min(width, self.local), dim=-1)
        vals = self.comm.all_gather_last(v.float().contiguous())                      # [M, tp * width]
        ids = self.comm.all_gather_last((local + self.offset).contiguous())
        top_v, top = vals.topk(min(width, vals.shape[1]), dim=-1)
        cand = ids.gather(-1, top)
        if self.rescore:
            mine = (cand >= self.offset) & (cand < self.offset + self.local)
            rows = self.shard[(cand - self.offset).clamp(0, self.local - 1)].float()
            exact = torch.bmm(rows, flat.float().unsqueeze(-1)).squeeze(-1) * mine
            exact = self.comm.all_reduce(exact)
            top_v, order = exact.topk(r, dim=-1)
            cand = cand.gather(-1, order)
        return cand[:, :r].reshape(*x.shape[:-1], r), top_v[:, :r].reshape(*x.shape[:-1], r)

    def argmax(self, x: torch.Tensor) -> torch.Tensor:
        ids, _ = self.candidates(x, 1)
        return ids[..., 0]

    def argmax_confidence(self, x: torch.Tensor):
        """The argmax and the softmax top-1 probability and margin over the whole vocabulary, from every rank's
        log-sum-exp and best two."""
        flat = x.reshape(-1, x.shape[-1])
        lg = self._logits(flat).float()
        stats = torch.cat([torch.logsumexp(lg, -1, keepdim=True), lg.topk(2, dim=-1).values], -1)
        stats = self.comm.all_gather_last(stats.contiguous()).view(flat.shape[0], -1, 3)
        lse = torch.logsumexp(stats[..., 0], -1)
        top = stats[..., 1:].reshape(flat.shape[0], -1).topk(2, dim=-1).values
        probs = torch.exp(top - lse.unsqueeze(-1))
        conf = torch.stack([probs[:, 0], probs[:, 0] - probs[:, 1]], -1)
        return self.argmax(x), conf.view(*x.shape[:-1], 2)


def make_draft_head(model, comm=None, fmt: str = "target", ids: Optional[torch.Tensor] = None, rescore: int = -1):
    """`fmt` "target" (the model's own head), "bf16" (row subset) or "w3" (3-bit copy, rescored by default)."""
    if fmt == "target":
        return TargetHead(lambda x: model.logits(x, comm) if comm is not None else model.logits(x))
    rescore = DEFAULT_RESCORE.get(fmt, 0) if rescore < 0 else rescore
    if comm is not None and getattr(model, "vocab_shard", 0):
        return VocabParallelHead(model.lm_head, comm, model.target.tp_rank, fmt, rescore)
    return ShortlistHead(model.lm_head, ids, fmt, rescore)
