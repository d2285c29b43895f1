"""Proposer construction by name. MAX_DEPTHS bounds the verify graphs captured per proposer kind
(reference: hibana/proposers/factory.py, MAX_DEPTHS = {"mtp": 8, "dflash2": 15})."""
from __future__ import annotations

import torch

MAX_DEPTHS = {"mtp": 8, "ngram": 15, "dflash2": 15, "lilicorr": 15}


def make_proposer(kind: str, executor=None, **kw):
    if kind == "ngram":
        from .ngram import NgramProposer
        return NgramProposer(**kw)
    if kind == "mtp":
        from ..engine.spec import SpecDecoder
        if executor is None or executor.model.mtp is None:
            raise ValueError("the MTP proposer needs a model with an MTP head")
        return SpecDecoder(executor, depth=kw.get("depth", 2))
    if kind == "lilicorr":
        from ..models.lilicorr import LiLiCorrDrafter
        from .parallel import ParallelProposer
        if executor is None:
            raise ValueError("the LiLiCorr drafter shares the target's embedding and output head: pass the executor")
        model = executor.model
        t = model.target
        drafter = kw.pop("drafter", None) or LiLiCorrDrafter(
            t.hidden, t.vocab, model.embed, model.lm_head, device=model.device,
            dtype=torch.float32 if str(model.device) == "cpu" else torch.bfloat16, **kw)
        return ParallelProposer(drafter)
    if kind in ("dflash2", "parallel"):
        from ..models.parallel_draft import BlockDrafter
        from .parallel import ParallelProposer
        if executor is None:
            raise ValueError("the block drafter shares the target's embedding and output head: pass the executor")
        model = executor.model
        t = model.target
        drafter = kw.pop("drafter", None) or BlockDrafter(
            t.hidden, t.vocab, model.embed, model.lm_head, device=model.device,
            dtype=torch.float32 if str(model.device) == "cpu" else torch.bfloat16, **kw)
        return ParallelProposer(drafter)
    raise ValueError(f"unknown proposer '{kind}' (known: {sorted(MAX_DEPTHS)})")
