"""Settings resolution: target defaults < profile defaults < config file < HIBANA_* environment < command-line flags.

Produces one `EngineConfig`; cross-field checks reject combinations the engine cannot serve.
Reference: hibana/launch/settings.py:35-523 (TARGET_SETTINGS, profile_defaults, resolve, _check).
"""
from __future__ import annotations

import dataclasses
import os
from pathlib import Path
from typing import Optional

from ..config import EngineConfig
from ..target import PRESETS, get_target

ALIASES = {"27b": "qwen38", "qwen": "qwen38", "flash-next": "flashnext", "fn": "flashnext", "super": "nemotron",
           "dense": "dense-27b", "tiny": "tiny-hybrid-moe"}

TARGET_SETTINGS = {
    "dense-27b": {"port": 30001, "max_batch": 64, "prefill_chunk": 2048},
    "qwen38": {"port": 30001, "max_batch": 64, "prefill_chunk": 2048, "spec": "mtp"},
    "flashnext": {"port": 30004, "max_batch": 128, "prefill_chunk": 4096, "spec": "mtp", "ep": 8, "tp": 8},
    "nemotron": {"port": 30005, "max_batch": 128, "prefill_chunk": 4096, "spec": "mtp", "ep": 8, "tp": 8},
    "bolt": {"port": 30007, "max_batch": 16, "prefill_chunk": 2048, "spec": "lilicorr", "spec_depth": 4},
    "tiny-hybrid-moe": {"port": 30006, "max_batch": 8, "prefill_chunk": 256, "spec": "mtp", "spec_depth": 2},
    "dense-tiny": {"port": 30006, "max_batch": 8, "prefill_chunk": 512},
}


def profile_defaults(profile: str) -> dict:
    """exact: bitwise-greedy speculation; fast: relaxed acceptance and deeper drafts; throughput: large batches,
    quantised recurrent state, no speculation at high load."""
    if profile == "exact":
        return {"accept_top_k": 1, "accept_margin": 0.0, "spec_depth": 3}
    if profile == "fast":
        return {"accept_top_k": 2, "accept_margin": 1.0, "spec_depth": 4, "accept_soft": 0.5}
    if profile == "throughput":
        return {"max_batch": 256, "spec_depth": 1, "ssm_state": "int8", "prefill_budget": 8192,
                "graph_buckets": "1,2,4,8,16,32,64,128,256"}
    raise ValueError(f"unknown profile {profile!r}")


def read_config_file(path: Optional[str]) -> dict:
    """KEY=VALUE lines (HIBANA_ prefix optional); '#' starts a comment."""
    candidates = [path] if path else [os.environ.get("HIBANA_CONFIG_FILE"),
                                      str(Path.home() / ".config" / "hibana" / "hibana.env")]
    out = {}
    for c in candidates:
        if c and Path(c).exists():
            for line in Path(c).read_text().splitlines():
                line = line.split("#", 1)[0].strip()
                if "=" in line:
                    k, v = line.split("=", 1)
                    k = k.strip()
                    out[k if k.startswith(("HIBANA_", "SHARAR_")) else "HIBANA_" + k.upper()] = v.strip().strip('"')
            break
    return out


def _check(cfg: EngineConfig) -> None:
    t = get_target(cfg.target)
    if cfg.tp > 1:
        for v, name in ((t.q_heads, "q heads"), (t.ffn, "ffn"), (t.mamba_heads, "mamba heads"),
                        (t.gdn_k_heads, "gdn k heads")):
            if v and v % cfg.tp:
                raise ValueError(f"{t.name}: {name} = {v} does not divide by tp = {cfg.tp}")
    if cfg.ep > 1 and not t.experts:
        raise ValueError(f"{t.name} has no experts: ep must be 1")
    if cfg.ep > 1 and t.experts % cfg.ep:
        raise ValueError(f"{t.experts} experts do not divide by ep = {cfg.ep}")
    if cfg.spec == "mtp" and not t.mtp_layers:
        raise ValueError(f"{t.name} has no MTP head")
    if cfg.ssd_dir and not cfg.radix_cache:
        raise ValueError("the SSD tier needs the radix cache")


def resolve(target: Optional[str] = None, *, profile: Optional[str] = None, config_file: Optional[str] = None,
            env: Optional[dict] = None, flags: Optional[dict] = None) -> EngineConfig:
    env = dict(os.environ if env is None else env)
    file_env = read_config_file(config_file)
    merged_env = {**file_env, **{k: v for k, v in env.items() if k.startswith(("HIBANA_", "SHARAR_"))}}
    name = target or merged_env.get("HIBANA_TARGET") or "dense-27b"
    name = ALIASES.get(name, name)
    if name not in PRESETS:
        raise ValueError(f"unknown target {name!r}; known: {sorted(set(PRESETS) | set(ALIASES))}")
    name = get_target(name).name if name not in TARGET_SETTINGS else name
    prof = profile or merged_env.get("HIBANA_PROFILE") or "exact"
    values = {"target": name, "profile": prof}
    values.update(TARGET_SETTINGS.get(name, {}))
    if "tp" in values or "ep" in values:        # multi-GPU defaults apply only when the GPUs exist
        try:
            import torch
            n = torch.cuda.device_count()
        except Exception:  # noqa: BLE001
            n = 0
        if n < values.get("tp", 1):
            values["tp"] = 1
            values["ep"] = 1
    values.update(profile_defaults(prof))
    fields = {f.name for f in dataclasses.fields(EngineConfig)}
    cfg = EngineConfig.from_env(merged_env, **{k: v for k, v in values.items() if k in fields
                                               and "HIBANA_" + k.upper() not in merged_env})
    if flags:
        cfg = cfg.replace(**{k: v for k, v in flags.items() if v is not None and k in fields})
    _check(cfg)
    return cfg
