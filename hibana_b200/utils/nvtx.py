"""NVTX ranges around the engine's phases (scheduler step, prefill chunk, decode step, speculative round, SSD
restore), so that a timeline capture shows which kernels belong to what. Off unless `EngineConfig.nvtx` is set: a
disabled range costs one attribute read. Reference: hibana/engine/executor.py (torch.cuda.nvtx ranges under
HIBANA_NVTX)."""
from __future__ import annotations

import contextlib

import torch

from .. import config as cfgmod

OPEN: list[str] = []          # names of the ranges opened so far (tests read it; bounded)


@contextlib.contextmanager
def span(name: str):
    if not cfgmod.current().nvtx:
        yield
        return
    if len(OPEN) < 4096:
        OPEN.append(name)
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on_gpu:
            torch.cuda.nvtx.range_pop()


def ranged(name: str):
    """Decorator form of `span`."""
    def wrap(fn):
        def inner(*a, **kw):
            if not cfgmod.current().nvtx:
                return fn(*a, **kw)
            with span(name):
                return fn(*a, **kw)
        inner.__name__, inner.__doc__, inner.__wrapped__ = fn.__name__, fn.__doc__, fn
        return inner
    return wrap
