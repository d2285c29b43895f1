"""Engine settings: one frozen dataclass, one field per `HIBANA_*` variable, read through `current()`.

No other module reads the environment for engine behaviour; tests install a config with `using(...)`.
Mirrors the control-plane rule of the reference (hibana/engine/config.py:83-274) with the fields this engine has:
tensor / expert / data parallel sizes up to 8 GPUs, peer-memory communicator switches, pool sizing.
"""
from __future__ import annotations

import contextlib
import dataclasses
import os
from dataclasses import dataclass
from typing import Iterator, Optional

from .hardware.b200 import HOST_FLOOR_GIB


def _bool(v: str) -> bool:
    return v.strip().lower() in ("1", "true", "yes", "on")


@dataclass(frozen=True)
class EngineConfig:
    # model / serving
    target: str = "dense-27b"
    profile: str = "exact"                 # exact | fast | throughput
    weights: str = "random"                # random | path to a checkpoint directory
    seed: int = 0
    max_batch: int = 64
    max_context: int = 0                   # 0 = target default
    max_queue: int = 256
    # parallelism (one process per GPU)
    tp: int = 1
    ep: int = 1
    dp: int = 1
    fused_collectives: bool = True         # peer-memory fused kernels; False = NCCL-only baseline path
    comm_timeout_ms: int = 2000            # bound of every device-side wait on a peer
    comm_buffer_mb: int = 64
    control_timeout_s: int = 30            # host control plane: broadcast timeout and peer-heartbeat limit
    # scheduler
    prefill_chunk: int = 0                 # 0 = target default
    prefill_budget: int = 4096
    decode_reserve: int = 64
    decode_steps_per_chunk: int = 1
    max_waits: int = 8
    # memory
    gpu_memory_fraction: float = 0.90
    host_floor_gib: float = HOST_FLOOR_GIB # free host memory left to the OS; the memory guard stops the engine when
                                           # it stays under half of this (0 = no guard) (launch/guard.py)
    kv_pages: int = 0                      # 0 = plan from free memory
    state_slots: int = 0
    kv_dtype: str = ""                     # "" = target default, else bf16 | fp8 | nvfp4 (4.5 bits per element)
    ssm_state: str = "fp32"                # fp32 | fp16_sr | int8 | int8w (int8 boundary state + window of records,
                                           # Mamba-2 and delta-rule layers; ops/ssm_window.py)
    ssm_window: int = 16                   # committed tokens between two quantisations of an int8w state
    # prefix cache / SSD tier
    radix_cache: bool = True
    ssd_dir: str = ""
    ssd_budget_gb: float = 200.0
    ssd_min_prefix: int = 4096
    ssd_min_gain: int = 2048
    ssd_block_tokens: int = 256
    # speculation
    spec: str = "off"                      # off | mtp | dflash2 | ngram | lilicorr
    spec_depth: int = 3
    spec_depths: str = ""                  # per-bucket depths "1:4,8:3,64:1"
    spec_state: str = "reconstruct"        # snapshots | reconstruct
    accept_top_k: int = 1
    accept_margin: float = 0.0
    accept_soft: float = 0.0
    device_accept: bool = True
    # graphs
    cuda_graphs: bool = True
    graph_buckets: str = "1,2,4,8,16,32,64,128,256"
    # kernels / numerics
    w3: bool = False
    w3_checkpoint: str = ""                # calibrated decode copies to attach over the nearest-rounded ones
                                           # (weights/calibrate_model.py)
    stable_numerics: bool = False
    attn_splits: int = 0                   # 0 = automatic
    gemv: bool = False                     # small NVFP4 projections of up to 4 rows take the register-decode GEMV
                                           # (ops/gemv.py); measured slower than the tcgen05 GEMM inside the 27B step
    fuse_epilogues: bool = True            # requantise / merge inside the producing kernel (decode shapes)
    fuse_attn_tail: bool = False           # decode attention merges its KV splits in its last-arriving CTA (measured
                                           # slower than the merge kernel at batch 64: off; the merge kernel then
                                           # writes the NVFP4 rows, and an unsplit launch always quantises in-kernel)
    decode_attn: str = "mma"               # mma | tc (persistent tcgen05 kernel, head dim 128)
    prefill_attn: str = "tc"               # tc | general
    gdn_phase1: str = "cuda"               # cuda | torch
    ssd_phase1: str = "cuda"               # cuda | torch
    gemm_local_reduce: bool = True         # unsplit decode tiles: epilogue through the parked partial (wide stores)
    attn_ctas_per_sm: int = 1              # CTA slots per SM assumed when choosing KV splits (the kernel runs two per
                                           # SM, but modelling both measured slower: more splits, more partials to merge)
    max_splits: int = 8                    # split-K cluster size cap (8 = portable)
    pdl: int = 1                           # programmatic dependent launch level (0 off, 1 GEMMs, 2 small kernels too)
    overlap_rows: int = 64                 # up to this many rows a MoE layer's independent chains (shared expert,
                                           # latent projection) run on a side stream beside the routed experts; 0 = off
    expert_budget: int = 0                 # > 0: decode-sized MoE calls read at most this many distinct experts
    expert_keep: int = 2                   # with a budget: choices of every row that are always honoured
    # observability
    trace_dir: str = ""
    trace_cap_gb: float = 32.0
    debug_sync: bool = False
    bounds: bool = False                   # load the checked-index build of the native library (debugging; slower)
    ssd_trace: bool = False                # one JSON line per SSD restore / backup in <trace_dir or ssd_dir>/ssd_trace.jsonl
    nvtx: bool = False                     # NVTX ranges around scheduler steps, prefill chunks, decode steps, rounds
    # api
    host: str = "127.0.0.1"
    port: int = 30001
    api_key: str = ""

    def __post_init__(self) -> None:
        if self.tp not in (1, 2, 4, 8) or self.ep not in (1, 2, 4, 8) or self.dp not in (1, 2, 4, 8):
            raise ValueError("tp, ep and dp must each be 1, 2, 4 or 8")
        if self.tp * self.dp > 8:
            raise ValueError("tp * dp must fit one 8-GPU box")
        if self.ep > 1 and self.ep != self.tp * self.dp and self.ep != self.tp:
            raise ValueError("ep must equal tp or tp * dp (experts are sharded over the same ranks)")
        if self.profile not in ("exact", "fast", "throughput"):
            raise ValueError(f"unknown profile {self.profile!r}")
        if self.spec not in ("off", "mtp", "dflash2", "ngram", "lilicorr"):
            raise ValueError(f"unknown spec {self.spec!r}")
        if self.spec_state not in ("snapshots", "reconstruct"):
            raise ValueError(f"unknown spec_state {self.spec_state!r}")
        if not 0.05 <= self.gpu_memory_fraction <= 0.98:
            raise ValueError("gpu_memory_fraction out of range")
        if self.max_batch < 1 or self.max_batch > 1024:
            raise ValueError("max_batch out of range")

    @property
    def buckets(self) -> tuple[int, ...]:
        out = sorted({int(b) for b in self.graph_buckets.split(",") if b.strip()})
        return tuple(b for b in out if b <= max(self.max_batch, 1)) or (1,)

    @property
    def world(self) -> int:
        return self.tp * self.dp

    @classmethod
    def from_env(cls, env: Optional[dict] = None, **overrides) -> "EngineConfig":
        env = os.environ if env is None else env
        values = {}
        for f in dataclasses.fields(cls):
            raw = env.get("HIBANA_" + f.name.upper())
            if raw is None:
                raw = env.get("SHARAR_" + f.name.upper())  # legacy prefix
            if raw is None:
                continue
            if f.type in ("bool", bool):
                values[f.name] = _bool(raw)
            elif f.type in ("int", int):
                values[f.name] = int(raw)
            elif f.type in ("float", float):
                values[f.name] = float(raw)
            else:
                values[f.name] = raw
        values.update(overrides)
        return cls(**values)

    def replace(self, **kw) -> "EngineConfig":
        return dataclasses.replace(self, **kw)

    def as_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d["api_key"] = "***" if self.api_key else ""
        return d


_CURRENT: Optional[EngineConfig] = None


def current() -> EngineConfig:
    global _CURRENT
    if _CURRENT is None:
        _CURRENT = EngineConfig.from_env()
    return _CURRENT


def install(cfg: EngineConfig) -> EngineConfig:
    global _CURRENT
    _CURRENT = cfg
    return cfg


def reset() -> None:
    global _CURRENT
    _CURRENT = None


@contextlib.contextmanager
def using(cfg: Optional[EngineConfig] = None, **overrides) -> Iterator[EngineConfig]:
    """Temporarily installs `cfg` (or the current config with overrides)."""
    global _CURRENT
    prev = _CURRENT
    base = cfg if cfg is not None else (prev or EngineConfig())
    _CURRENT = base.replace(**overrides) if overrides else base
    try:
        yield _CURRENT
    finally:
        _CURRENT = prev
