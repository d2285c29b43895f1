"""Offline entry point: build a model + executor + scheduler from an `EngineConfig` and generate.

`LLM.generate(prompts, params)` is the public call a library user makes; the HTTP server builds the same stack and
drives it through the EngineLoop. Reference: hibana/engine/run.py (generate_cli), hibana/target.py:399 (load_model).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..config import EngineConfig, current
from ..target import Target, get_target
from .executor import Executor
from .request import Request, SamplingParams
from .scheduler import Scheduler, SchedulerConfig


def build_model(target: Target, device, seed: int = 0, comm=None):
    """Random-init model of the target's family (checkpoint loading goes through hibana_b200.weights)."""
    if target.family == "dense":
        from ..models.dense import DenseModel
        return DenseModel(target, device, seed=seed)
    from ..models.hybrid import HybridModel
    return HybridModel(target, device, seed=seed)


class LLM:
    def __init__(self, cfg: Optional[EngineConfig] = None, *, target: Optional[Target] = None, device=None,
                 model=None, max_ctx: Optional[int] = None, comm=None):
        self.cfg = cfg or current()
        self.target = target or get_target(self.cfg.target)
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.model = model or build_model(self.target, self.device, self.cfg.seed, comm)
        ctx = max_ctx or self.cfg.max_context or min(self.target.max_context, 8192)
        self.executor = Executor(self.model, max_batch=self.cfg.max_batch, max_ctx=ctx,
                                 kv_slots=self.cfg.kv_pages, use_graphs=self.cfg.cuda_graphs,
                                 buckets=self.cfg.buckets, radix_cache=self.cfg.radix_cache, comm=comm,
                                 attn_splits=self.cfg.attn_splits, decode_reserve=self.cfg.decode_reserve)
        self.scheduler = Scheduler(self.executor, SchedulerConfig(
            prefill_chunk=self.cfg.prefill_chunk or self.target.prefill_chunk,
            prefill_budget=self.cfg.prefill_budget, max_batch=self.cfg.max_batch, max_queue=self.cfg.max_queue,
            decode_steps_per_chunk=self.cfg.decode_steps_per_chunk, max_waits=self.cfg.max_waits))
        if self.cfg.cuda_graphs and self.device.type == "cuda":
            self.executor.capture_graphs()

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: SamplingParams | Sequence[SamplingParams] = SamplingParams()) -> list[Request]:
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        reqs = [self.scheduler.submit(Request(prompt_ids=list(p), params=sp)) for p, sp in zip(prompts, plist)]
        while not self.scheduler.idle():
            self.scheduler.step()
        return reqs
