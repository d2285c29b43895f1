"""Per-rank model snapshots: every tensor a model holds, by attribute path, in safetensors shards.

`save_state(model, directory)` walks the model object (layers, linears, quantised tensors, expert stacks, norms,
convolution and recurrence parameters, drafter heads) and writes each tensor under its attribute path
(`blocks.3.mixer.in_qkvz.wq.q`, `blocks.5.ffn.experts.fc1.sf`, ...); `load_state(model, directory)` puts them back
into a model of the same structure, bit for bit (packed NVFP4 values, swizzled scales, per-tensor scales and
calibrated activation scales included). Under tensor parallelism each rank writes and reads its own shard
directory `rank<r>of<n>/`, so a rank touches only the bytes it keeps. This is the engine's own format for every
model family; published dense checkpoints with separate projections load through weights/checkpoint.py.
Reference: hibana/weights/safetensors.py:1-61 (lazy per-file access), hibana/target.py:399 (load_model).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator

import torch
from safetensors import safe_open
from safetensors.torch import save_file

import types

INDEX = "model.safetensors.index.json"
_NOT_STATE = (types.FunctionType, types.MethodType, types.ModuleType, type)
_SKIP = {"target", "full", "t", "device", "base", "_vision", "vision_cfg", "hyper_sites_cache"}


def _walk(obj, prefix: str, seen: set) -> Iterator[tuple]:
    """Yields (path, holder, key) for every tensor reachable from `obj` (holder[key] / getattr(holder, key))."""
    if id(obj) in seen:
        return
    seen.add(id(obj))
    if isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            if isinstance(v, torch.Tensor):
                yield f"{prefix}{i}", obj, i
            elif hasattr(v, "__dict__") or isinstance(v, (list, tuple, dict)):
                yield from _walk(v, f"{prefix}{i}.", seen)
        return
    if isinstance(obj, dict):
        for k, v in obj.items():
            if isinstance(v, torch.Tensor):
                yield f"{prefix}{k}", obj, k
            elif hasattr(v, "__dict__") or isinstance(v, (list, tuple, dict)):
                yield from _walk(v, f"{prefix}{k}.", seen)
        return
    for k, v in vars(obj).items():
        if k in _SKIP or k.startswith("__"):
            continue
        if isinstance(v, torch.Tensor):
            yield f"{prefix}{k}", obj, k
        elif isinstance(v, (list, tuple, dict)) or (hasattr(v, "__dict__") and not isinstance(v, _NOT_STATE)
                                                     and type(v).__module__.startswith("hibana_b200")):
            yield from _walk(v, f"{prefix}{k}.", seen)


def named_tensors(model) -> dict:
    out = {}
    for path, holder, key in _walk(model, "", set()):
        t = holder[key] if isinstance(holder, (list, dict)) else getattr(holder, key)
        out[path] = (holder, key, t)
    return out


def _rank_dir(directory: str, rank: int, tp: int) -> Path:
    d = Path(directory)
    return d / f"rank{rank}of{tp}" if tp > 1 else d


def save_state(model, directory: str, max_shard_bytes: int = 4 << 30) -> dict:
    t = model.target
    d = _rank_dir(directory, t.tp_rank, t.tp_size)
    d.mkdir(parents=True, exist_ok=True)
    items = named_tensors(model)
    shards, cur, size = [], {}, 0
    seen_storage: dict = {}
    alias = {}
    for name, (_, _, tensor) in items.items():
        key = (tensor.data_ptr(), tuple(tensor.shape), tensor.dtype) if tensor.numel() else None
        if key is not None and key in seen_storage:          # tied tensors (lm_head = embed) are stored once
            alias[name] = seen_storage[key]
            continue
        if key is not None:
            seen_storage[key] = name
        x = tensor.detach().cpu().contiguous()
        if x.dtype == torch.bool:
            x = x.to(torch.uint8)
        nbytes = x.numel() * x.element_size()
        if cur and size + nbytes > max_shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[name] = x
        size += nbytes
    if cur:
        shards.append(cur)
    index = {}
    for i, shard in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, str(d / fname))
        index.update({k: fname for k in shard})
    meta = {"format": "hibana-b200-snapshot", "target": t.name, "tp_size": t.tp_size, "tp_rank": t.tp_rank,
            "family": t.family, "layers": len(t.layers), "hidden": t.hidden, "weight_format": t.weight_format}
    (d / INDEX).write_text(json.dumps({"metadata": meta, "weight_map": index, "aliases": alias}, indent=1))
    if t.tp_size > 1 and t.tp_rank == 0:
        (Path(directory) / INDEX).write_text(json.dumps({"metadata": dict(meta, sharded=True), "weight_map": {}}))
    return meta


def load_state(model, directory: str, strict: bool = True) -> int:
    """Overwrites the model's tensors with the stored ones (same paths, shapes and dtypes). Returns the count."""
    t = model.target
    d = _rank_dir(directory, t.tp_rank, t.tp_size)
    idx = json.loads((d / INDEX).read_text())
    meta = idx.get("metadata", {})
    if meta.get("format") != "hibana-b200-snapshot":
        raise ValueError(f"{d} is not a snapshot of this engine")
    for k in ("tp_size", "layers", "hidden", "family"):
        want = {"tp_size": t.tp_size, "layers": len(t.layers), "hidden": t.hidden, "family": t.family}[k]
        if meta.get(k) != want:
            raise ValueError(f"snapshot {k} = {meta.get(k)!r} does not match the model's {want!r}")
    files: dict = {}
    items = named_tensors(model)
    n = 0
    wmap, aliases = idx["weight_map"], idx.get("aliases", {})
    for name, (holder, key, tensor) in items.items():
        src = aliases.get(name, name)
        if src not in wmap:
            if strict:
                raise KeyError(f"snapshot has no tensor {name!r}")
            continue
        f = wmap[src]
        if f not in files:
            files[f] = safe_open(str(d / f), framework="pt", device="cpu")
        x = files[f].get_tensor(src)
        if tuple(x.shape) != tuple(tensor.shape):
            raise ValueError(f"{name}: stored shape {tuple(x.shape)} != model shape {tuple(tensor.shape)}")
        tensor.copy_(x.to(tensor.dtype) if x.dtype != tensor.dtype else x)
        n += 1
    return n


def is_snapshot(directory: str) -> bool:
    p = Path(directory) / INDEX
    if not p.exists():
        return False
    try:
        return json.loads(p.read_text()).get("metadata", {}).get("format") == "hibana-b200-snapshot"
    except (OSError, ValueError):
        return False
