"""Offline entry point: build a model + executor + scheduler from an `EngineConfig` and generate.

`LLM.generate(prompts, params)` is the public call a library user makes; the HTTP server builds the same stack and
drives it through the EngineLoop. Everything a setting can switch is wired here, once: the checkpoint (`weights`),
the memory plan that sizes the KV and recurrent-state pools from the memory left beside the weights
(`gpu_memory_fraction`, `kv_pages`, `state_slots`, `max_context`), KV / state formats (`kv_dtype`, `ssm_state`),
the SSD tier (`ssd_dir` and its limits), speculation (`spec`, `spec_depth`), graphs and their warm-up, and
`debug_sync`. Reference: hibana/engine/run.py (generate_cli), hibana/target.py:399 (load_model),
hibana/engine/executor.py:51-181,300-309,356-422 (memory plan, warmup, enable_ssd_tier, persist_prefixes).
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence

import torch

from ..cache import ledger
from ..config import EngineConfig, current
from ..target import Target, get_target
from .executor import Executor
from .request import Request, SamplingParams
from .scheduler import Scheduler, SchedulerConfig

STATE_DTYPES = {"fp32": torch.float32, "fp16_sr": torch.float16, "int8": torch.int8, "int8w": torch.int8}
KV_DTYPES = {"bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn, "nvfp4": "nvfp4"}


def checkpoint_dir(weights: str) -> Optional[str]:
    """The directory of `weights` when it names a checkpoint this engine can read, else None (random init)."""
    if not weights or weights == "random":
        return None
    from ..weights.checkpoint import INDEX
    if (Path(weights) / INDEX).exists():
        return weights
    raise FileNotFoundError(f"{weights!r} is not a checkpoint directory (no {INDEX})")


def build_model(target: Target, device, seed: int = 0, comm=None, weights: str = "random", tp: int = 1,
                rank: int = 0, ep: int = 1):
    """The target's model: loaded from the checkpoint directory `weights` (this rank's tensor-parallel shard is
    cut out of the stored tensors), or random-init N(0, 0.02) from `seed` when `weights` is "random". `ep` > 1
    (with tp == 1): a data-parallel replica that keeps experts [rank * E / ep, (rank + 1) * E / ep) of every MoE
    layer and everything else whole."""
    ckpt = checkpoint_dir(weights)
    if ep > 1 and tp == 1:
        if ckpt is not None:
            raise NotImplementedError("expert-parallel replicas start from random weights or a per-rank snapshot")
        if not target.experts or target.experts % ep:
            raise ValueError(f"{target.name}: {target.experts} experts do not divide over ep={ep}")
        from ..models.hybrid import HybridModel
        return HybridModel(target, device, seed=seed, ep_rank=rank, ep_size=ep)
    if target.family == "dense":
        from ..models.dense import DenseModel
        from ..weights import snapshot
        if ckpt is not None and snapshot.is_snapshot(ckpt):
            model = DenseModel(target, device, seed=seed) if tp == 1 else DenseModel.sharded(target, tp, rank, device, seed)
            snapshot.load_state(model, ckpt)
            return model
        if ckpt is not None:
            from ..weights.checkpoint import load_dense
            return load_dense(target, ckpt, device, tp=tp, rank=rank)
        return DenseModel(target, device, seed=seed) if tp == 1 else DenseModel.sharded(target, tp, rank, device, seed)
    from ..models.hybrid import HybridModel
    if ckpt is not None:
        from ..weights.checkpoint import load_hybrid
        return load_hybrid(target, ckpt, device, tp=tp, rank=rank)
    if tp > 1:
        return HybridModel.sharded(target, tp, rank, device, seed=seed)
    return HybridModel(target, device, seed=seed)


def plan_memory(cfg: EngineConfig, target: Target, device: torch.device, *, max_ctx: Optional[int] = None,
                free_bytes: Optional[int] = None, comm_bytes: int = 0, kv_layers: Optional[int] = None) -> dict:
    """Pool sizes for this process: {max_ctx, kv_slots, state_slots, plan}. On a CUDA device the pools take what
    the ledger leaves of the memory that is free AFTER the weights were loaded; explicit `kv_pages` / `state_slots`
    win. Without a device (CPU tests) the pools are just large enough for max_batch x max_ctx."""
    tp = max(target.tp_size, 1)
    esz = {"bf16": 2, "fp8": 1, "nvfp4": 0.5625}[cfg.kv_dtype or target.kv_dtype]     # nvfp4: 4 bits + a scale per 16
    layers = target.attn_layers + (1 if target.mtp_layers else 0) if kv_layers is None else kv_layers
    kv_tok = int(layers * 2 * max(target.kv_heads, 1) * target.head_dim * esz)
    state_slot = target.state_bytes_per_slot
    if cfg.ssm_state != "fp32" and state_slot:
        # fp16: half; int8: a quarter + row scales; int8w: a quarter + the window's records (about 0.6 of that again)
        div = {"fp16_sr": 2.0, "int8": 4.0, "int8w": 2.4}.get(cfg.ssm_state, 4.0)
        state_slot = int(state_slot / div) + target.recurrent_layers * 4096
    if device.type != "cuda" and free_bytes is None:
        ctx = max_ctx or cfg.max_context or min(target.max_context, 8192)
        return {"max_ctx": ctx, "kv_slots": cfg.kv_pages, "state_slots": cfg.state_slots, "plan": None}
    if free_bytes is None:
        free_bytes = torch.cuda.mem_get_info(device)[0]
    ctx = max_ctx or cfg.max_context or target.max_context
    buckets = cfg.buckets
    graph = ledger.graph_bytes(buckets, target.hidden, target.vocab // tp, len(target.layers)) if cfg.cuda_graphs else 0
    chunk = cfg.prefill_chunk or target.prefill_chunk
    act = ledger.activation_bytes(max(chunk, cfg.prefill_budget), target.hidden, max(target.ffn, target.expert_ffn * 8),
                                  max(target.q_heads, 1) * target.head_dim, cfg.max_batch, target.vocab // tp)
    # block table (int32 per position and row) + split-KV partials of the widest bucket
    workspace = (cfg.max_batch + 1) * ctx * 4 + comm_bytes + cfg.max_batch * max(target.q_heads, 1) * target.head_dim * 4 * 16
    if cfg.spec != "off":      # what the speculator allocates after the pools exist is set aside now
        from ..cache.spec_budget import SpecConfig, budget
        spec_fixed, spec_slot = budget(SpecConfig(cfg.spec, cfg.spec_depth, cfg.spec_state), cfg.max_batch, target,
                                       buckets=len(cfg.buckets))
        workspace += spec_fixed
        if kv_layers is not None:      # the caller counted the model's KV layers without the drafter's
            kv_tok += spec_slot
    led = ledger.Ledger(free_bytes, fraction=cfg.gpu_memory_fraction)
    notes = []
    while True:
        try:
            plan = led.plan(kv_bytes_per_token=kv_tok, state_bytes_per_slot=state_slot, max_batch=cfg.max_batch,
                            max_ctx=ctx, graph=graph, workspace=workspace, activations=act,
                            want_state_slots=cfg.state_slots, ssd_restore=bool(cfg.ssd_dir))
            break
        except MemoryError:
            if ctx <= 2048 or cfg.max_context:      # an explicit context limit is a requirement, not a wish
                raise
            ctx //= 2                               # the target's native context does not fit beside the weights
            workspace = (cfg.max_batch + 1) * ctx * 4 + comm_bytes
            notes.append(f"context limit reduced to {ctx} tokens to fit the KV pool")
    plan.notes.extend(notes)
    return {"max_ctx": ctx, "kv_slots": cfg.kv_pages or plan.kv_slots, "state_slots": cfg.state_slots or plan.state_slots,
            "plan": plan}


class LLM:
    def __init__(self, cfg: Optional[EngineConfig] = None, *, target: Optional[Target] = None, device=None,
                 model=None, max_ctx: Optional[int] = None, comm=None, warmup: bool = False, control=None,
                 rank: Optional[int] = None):
        """`comm`: tensor-parallel communicator (cfg.tp ranks run the same requests). `control` + `rank`: this
        process is replica `rank` of cfg.dp data-parallel replicas and `control(obj) -> list` all-gathers small
        host objects between them (engine/dp.py); with cfg.ep == cfg.dp the replicas share every MoE layer's experts
        through the all-to-all of parallel/ep.py and run their forwards together. Both: replica `rank` is a
        tensor-parallel group; `control` goes to the group's rank 0 only."""
        self.cfg = cfg = cfg or current()
        full = target or get_target(cfg.target)
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        tp = comm.world if comm is not None and cfg.tp > 1 else 1
        self.lockstep = self.ep = None
        if cfg.dp > 1:
            if tp > 1 and cfg.ep not in (1, cfg.tp):
                raise NotImplementedError("expert parallelism across data-parallel replicas of tensor-parallel "
                                          "groups is not supported (experts shard inside a group: ep = tp)")
            # replicas of tensor-parallel groups: the group's rank 0 speaks for the replica, the others follow its
            # commands (engine/loop.py) and take no part in the replicas' rounds
            if not (tp > 1 and comm.rank != 0):
                if control is None or rank is None:
                    raise ValueError("dp > 1 needs the replicas' control all-gather and this replica's rank")
                from .dp import Lockstep
                self.lockstep = Lockstep(control, rank, cfg.dp)
        rank = comm.rank if comm is not None else (rank or 0)
        ep = cfg.ep if cfg.dp > 1 and tp == 1 and cfg.ep == cfg.dp else 1
        self.model = model or build_model(full, self.device, cfg.seed, comm, cfg.weights, tp=tp, rank=rank, ep=ep)
        self.target = self.model.target
        if cfg.w3 and hasattr(self.model, "attach_w3") and model is None:
            self.model.attach_w3()          # before the pools are sized: the copies take memory too
            if cfg.w3_checkpoint:
                from ..weights import calibrate_model
                calibrate_model.attach(self.model, cfg.w3_checkpoint)
        if ep > 1:
            self.ep = self._expert_parallel(ep, rank, control)
        mem = plan_memory(cfg, self.target, self.device, max_ctx=max_ctx,
                          comm_bytes=getattr(comm, "heap_bytes", 0) if comm is not None else 0,
                          kv_layers=getattr(self.model, "kv_layers", None) if getattr(self.model, "mtp", None) is None
                          else None)
        self.memory_plan = mem["plan"]
        self.executor = Executor(self.model, max_batch=cfg.max_batch, max_ctx=mem["max_ctx"],
                                 kv_slots=mem["kv_slots"], use_graphs=cfg.cuda_graphs,
                                 buckets=cfg.buckets, radix_cache=cfg.radix_cache, comm=comm,
                                 attn_splits=cfg.attn_splits, decode_reserve=cfg.decode_reserve,
                                 state_slots=mem["state_slots"],
                                 kv_dtype=KV_DTYPES[cfg.kv_dtype] if cfg.kv_dtype else None,
                                 state_dtype=STATE_DTYPES[cfg.ssm_state],
                                 state_window=cfg.ssm_window if cfg.ssm_state == "int8w" else 0,
                                 debug_sync=cfg.debug_sync)
        self.executor.runner.ep = self.ep          # before graphs are captured: the all-to-all is inside them
        if cfg.ssd_dir:
            self.executor.enable_ssd_tier(cfg.ssd_dir, budget_bytes=int(cfg.ssd_budget_gb * (1 << 30)),
                                          min_prefix=cfg.ssd_min_prefix, min_gain=cfg.ssd_min_gain,
                                          identity={"weights": cfg.weights, "seed": cfg.seed},
                                          trace_path=str(Path(cfg.trace_dir or cfg.ssd_dir) / "ssd_trace.jsonl")
                                          if cfg.ssd_trace else None)
            self.executor.rebuild_from_ssd()
        if cfg.spec == "mtp" and getattr(self.model, "mtp", None) is not None:
            self.executor.enable_spec(cfg.spec_depth)
        elif cfg.spec in ("dflash2", "ngram", "lilicorr"):       # drafts from a pluggable proposer (proposers/factory.py)
            self.executor.enable_spec(cfg.spec_depth, proposer=cfg.spec)
        self.scheduler = Scheduler(self.executor, SchedulerConfig(
            prefill_chunk=cfg.prefill_chunk or self.target.prefill_chunk,
            prefill_budget=cfg.prefill_budget, max_batch=cfg.max_batch, max_queue=cfg.max_queue,
            decode_steps_per_chunk=cfg.decode_steps_per_chunk, max_waits=cfg.max_waits))
        if cfg.cuda_graphs and self.device.type == "cuda":
            self.executor.capture_graphs()
        if warmup:
            self.executor.warmup()
        # graph capture and warm-up ran the same forwards on every replica; from here on they negotiate
        self.executor.runner.lockstep = self.lockstep

    def _expert_parallel(self, ep: int, rank: int, control):
        t, cfg = self.target, self.cfg
        width = t.latent or t.hidden
        if self.device.type != "cuda":
            from ..parallel.ep import HostExpertParallel
            return HostExpertParallel(control, rank, ep, t.experts)
        from ..parallel.ep import ExpertParallel
        depth = cfg.spec_depth + 1 if cfg.spec != "off" else 1
        tokens = max(cfg.prefill_budget, cfg.prefill_chunk or t.prefill_chunk, cfg.max_batch * depth)
        return ExpertParallel.create(rank, ep, self.device, tokens=tokens, topk=t.top_k, experts=t.experts,
                                     hidden=width, fmt="nvfp4" if t.weight_format == "nvfp4" else "bf16",
                                     timeout_ms=cfg.comm_timeout_ms)

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: SamplingParams | Sequence[SamplingParams] = SamplingParams()) -> list[Request]:
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        reqs = [self.scheduler.submit(Request(prompt_ids=list(p), params=sp)) for p, sp in zip(prompts, plist)]
        while not self.scheduler.idle():
            self.scheduler.step()
        if self.lockstep is not None:
            # other replicas may still be generating: keep joining their forwards until all have finished
            from .dp import LEAVING
            while any(s != LEAVING for s in self.executor.idle_round(LEAVING)):
                pass
        return reqs

    def shutdown(self) -> None:
        """Persists cached prefixes to the SSD tier (when enabled) and drains its writer."""
        self.executor.persist_prefixes()
