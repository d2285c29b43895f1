"""Proposer construction by name. MAX_DEPTHS bounds the verify graphs captured per proposer kind
(reference: hibana/proposers/factory.py, MAX_DEPTHS = {"mtp": 8, "dflash2": 15})."""
from __future__ import annotations

MAX_DEPTHS = {"mtp": 8, "ngram": 15}


def make_proposer(kind: str, executor=None, **kw):
    if kind == "ngram":
        from .ngram import NgramProposer
        return NgramProposer(**kw)
    if kind == "mtp":
        from ..engine.spec import SpecDecoder
        if executor is None or executor.model.mtp is None:
            raise ValueError("the MTP proposer needs a model with an MTP head")
        return SpecDecoder(executor, depth=kw.get("depth", 2))
    raise ValueError(f"unknown proposer '{kind}' (known: {sorted(MAX_DEPTHS)})")
