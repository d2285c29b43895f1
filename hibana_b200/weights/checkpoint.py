"""Save / load of the dense decoder as sharded safetensors files in the ModelOpt layout, with tensor-parallel
shards cut at load time (q/k/v by head, gate/up by column, o_proj/down by input feature) so that every rank reads
only the bytes it keeps. Names follow the Hugging Face convention of the family
(`model.layers.<i>.self_attn.qkv_proj`, `.o_proj`, `mlp.gate_up_proj`, `mlp.down_proj`, `input_layernorm`,
`post_attention_layernorm`, `model.embed_tokens`, `model.norm`, `lm_head`). An index file lists tensor -> file.
Reference: hibana/weights/safetensors.py:1-61 (SnapshotWeights), hibana/weights/sharding.py:1-88.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from ..models.dense import DenseModel
from ..models.linear import Linear
from ..target import Target
from . import modelopt

INDEX = "model.safetensors.index.json"


def _lin_tensors(lin: Linear, name: str) -> dict:
    if lin.fmt == "nvfp4":
        return modelopt.nvfp4_tensors(lin, name)
    return {f"{name}.weight": lin.weight.cpu().contiguous()}


def save_dense(model: DenseModel, directory: str, layers_per_file: int = 8) -> None:
    """Writes an UNSHARDED model (tp = 1)."""
    assert model.target.tp_size == 1
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    index, files = {}, []
    groups = [model.layers[i:i + layers_per_file] for i in range(0, len(model.layers), layers_per_file)]
    for gi, group in enumerate(groups):
        tensors = {}
        for layer in group:
            p = f"model.layers.{layer.idx}"
            tensors.update(_lin_tensors(layer.qkv, f"{p}.self_attn.qkv_proj"))
            tensors.update(_lin_tensors(layer.o, f"{p}.self_attn.o_proj"))
            tensors.update(_lin_tensors(layer.gate_up, f"{p}.mlp.gate_up_proj"))
            tensors.update(_lin_tensors(layer.down, f"{p}.mlp.down_proj"))
            tensors[f"{p}.input_layernorm.weight"] = layer.input_norm.cpu()
            tensors[f"{p}.post_attention_layernorm.weight"] = layer.post_norm.cpu()
        if gi == 0:
            tensors["model.embed_tokens.weight"] = model.embed.cpu()
            tensors["model.norm.weight"] = model.final_norm.cpu()
            if model.lm_head is not model.embed:
                tensors["lm_head.weight"] = model.lm_head.cpu()
        fname = f"model-{gi + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(d / fname))
        files.append(fname)
        index.update({k: fname for k in tensors})
    (d / INDEX).write_text(json.dumps({"metadata": {"format": "modelopt-nvfp4"}, "weight_map": index}, indent=1))


class Snapshot:
    """Lazy tensor access over the files of a checkpoint directory (only what is asked for is read)."""

    def __init__(self, directory: str):
        self.dir = Path(directory)
        self.map = json.loads((self.dir / INDEX).read_text())["weight_map"]
        self._open: dict = {}

    def __contains__(self, name: str) -> bool:
        return name in self.map

    def __getitem__(self, name: str) -> torch.Tensor:
        f = self.map[name]
        if f not in self._open:
            self._open[f] = safe_open(str(self.dir / f), framework="pt", device="cpu")
        return self._open[f].get_tensor(name)


def _load_lin(snap: Snapshot, name: str, device, rows=None, cols=None) -> Linear:
    if f"{name}.weight_scale" in snap:
        return modelopt.load_nvfp4_linear(snap, name, device, rows=rows, cols=cols)
    w = snap[f"{name}.weight"]
    if rows is not None:
        w = w[rows]
    if cols is not None:
        w = w[:, cols]
    return Linear(w.contiguous(), "bf16", name=name).to(device)


def load_dense(full: Target, directory: str, device="cpu", tp: int = 1, rank: int = 0) -> DenseModel:
    """Loads (a shard of) the model; shards are bitwise slices of the stored quantised matrices."""
    snap = Snapshot(directory)
    t = full.shard(tp, rank) if tp > 1 else full
    model = DenseModel.__new__(DenseModel)
    import math
    from ..ops import basic
    model.target, model.device = t, torch.device(device)
    d, hq, hkv = full.head_dim, full.q_heads // tp, max(full.kv_heads // tp, 1)
    kv0 = (rank * full.kv_heads) // tp
    f = full.ffn // tp
    model.layers = []
    for i in range(len(full.layers)):
        p = f"model.layers.{i}"
        layer = type("Layer", (), {})()
        layer.idx = i
        layer.input_norm = snap[f"{p}.input_layernorm.weight"].to(device)
        layer.post_norm = snap[f"{p}.post_attention_layernorm.weight"].to(device)
        if tp == 1:
            sel = ocols = gurows = dcols = None
        else:
            qrows = torch.arange(rank * hq * d, (rank + 1) * hq * d)
            krows = full.q_heads * d + torch.arange(kv0 * d, (kv0 + hkv) * d)
            vrows = (full.q_heads + full.kv_heads) * d + torch.arange(kv0 * d, (kv0 + hkv) * d)
            sel = torch.cat((qrows, krows, vrows))
            ocols = slice(rank * hq * d, (rank + 1) * hq * d)
            gurows = slice(2 * rank * f, 2 * (rank + 1) * f)
            dcols = slice(rank * f, (rank + 1) * f)
        layer.qkv = _load_lin(snap, f"{p}.self_attn.qkv_proj", device, rows=sel)
        layer.o = _load_lin(snap, f"{p}.self_attn.o_proj", device, cols=ocols)
        layer.gate_up = _load_lin(snap, f"{p}.mlp.gate_up_proj", device, rows=gurows)
        layer.down = _load_lin(snap, f"{p}.mlp.down_proj", device, cols=dcols)
        layer.linears = lambda layer=layer: [layer.qkv, layer.o, layer.gate_up, layer.down]
        model.layers.append(layer)
    model.embed = snap["model.embed_tokens.weight"].to(device)
    model.final_norm = snap["model.norm.weight"].to(device)
    head = snap["lm_head.weight"].to(device) if "lm_head.weight" in snap else model.embed
    model.vocab_shard = full.vocab // tp if tp > 1 and full.vocab % tp == 0 else 0
    model.lm_head = head[rank * model.vocab_shard:(rank + 1) * model.vocab_shard].contiguous() if model.vocab_shard else head
    model.inv_freq = basic.rope_inv_freq(t.rot_dim, t.rope_theta, device=model.device) if t.rot_dim else \
        torch.zeros(1, device=model.device)
    model.scale = 1.0 / math.sqrt(t.head_dim)
    model.kv_layers = len(model.layers)
    return model
