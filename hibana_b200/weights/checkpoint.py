"""Save / load of the dense decoder as sharded safetensors files in the ModelOpt layout, with tensor-parallel
shards cut at load time (q/k/v by head, gate/up by column, o_proj/down by input feature) so that every rank reads
only the bytes it keeps. Two layouts load: the Hugging Face / ModelOpt one with separate projections
(`model.layers.<i>.self_attn.{q,k,v,o}_proj`, `mlp.{gate,up,down}_proj`; q/k/v are concatenated and gate/up
interleaved pairwise at load, nothing is requantised) and this engine's pre-fused one (`self_attn.qkv_proj`,
`mlp.gate_up_proj`, rows already in kernel order). Both carry `input_layernorm`, `post_attention_layernorm`,
`model.embed_tokens`, `model.norm`, `lm_head`. An index file lists tensor -> file.
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


def _split_rows(lin: Linear, name_rows: list, deinterleave: bool = False) -> dict:
    """Tensors of the separate projections a fused Linear was built from: [(name, row selector)], or the even / odd
    rows when `deinterleave`."""
    out = {}
    if lin.fmt == "nvfp4":
        base = modelopt.nvfp4_tensors(lin, "x")
        for name, sel in name_rows:
            out[f"{name}.weight"] = base["x.weight"][sel].contiguous()
            out[f"{name}.weight_scale"] = base["x.weight_scale"].view(torch.uint8)[sel].contiguous().view(torch.float8_e4m3fn)
            out[f"{name}.weight_scale_2"] = base["x.weight_scale_2"].clone()
            out[f"{name}.input_scale"] = base["x.input_scale"].clone()
    else:
        for name, sel in name_rows:
            out[f"{name}.weight"] = lin.weight.cpu()[sel].contiguous()
    return out


def save_dense(model: DenseModel, directory: str, layers_per_file: int = 8, hf_layout: bool = False) -> None:
    """Writes an UNSHARDED model (tp = 1). `hf_layout` writes separate q/k/v and gate/up projections, the layout
    of published checkpoints; the default keeps the fused kernel-order matrices."""
    assert model.target.tp_size == 1
    t = model.target
    nq, nkv = t.q_heads * t.head_dim, t.kv_heads * t.head_dim
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    index, files = {}, []
    groups = [model.layers[i:i + layers_per_file] for i in range(0, len(model.layers), layers_per_file)]
    for gi, group in enumerate(groups):
        tensors = {}
        for layer in group:
            p = f"model.layers.{layer.idx}"
            if hf_layout:
                tensors.update(_split_rows(layer.qkv, [(f"{p}.self_attn.q_proj", slice(0, nq)),
                                                       (f"{p}.self_attn.k_proj", slice(nq, nq + nkv)),
                                                       (f"{p}.self_attn.v_proj", slice(nq + nkv, nq + 2 * nkv))]))
                tensors.update(_split_rows(layer.gate_up, [(f"{p}.mlp.gate_proj", slice(0, None, 2)),
                                                           (f"{p}.mlp.up_proj", slice(1, None, 2))]))
            else:
                tensors.update(_lin_tensors(layer.qkv, f"{p}.self_attn.qkv_proj"))
                tensors.update(_lin_tensors(layer.gate_up, f"{p}.mlp.gate_up_proj"))
            tensors.update(_lin_tensors(layer.o, f"{p}.self_attn.o_proj"))
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


def _load_fused(snap: Snapshot, names: list, device, parts=None, interleave: bool = False, name: str = "") -> Linear:
    """Separate stored projections -> one Linear (see modelopt.load_nvfp4_fused); bf16 sources are concatenated."""
    if f"{names[0]}.weight_scale" in snap:
        return modelopt.load_nvfp4_fused(snap, names, device, parts=parts, interleave=interleave, name=name)
    ws = []
    for i, n in enumerate(names):
        w = snap[f"{n}.weight"]
        ws.append(w if parts is None or parts[i] is None else w[parts[i]])
    if interleave:
        from ..models.linear import interleave_pairs
        w = interleave_pairs(ws[0], ws[1])
    else:
        w = torch.cat(ws, 0)
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
        if f"{p}.self_attn.qkv_proj.weight" in snap:
            layer.qkv = _load_lin(snap, f"{p}.self_attn.qkv_proj", device, rows=sel)
            layer.gate_up = _load_lin(snap, f"{p}.mlp.gate_up_proj", device, rows=gurows)
        else:
            # published layout: separate projections, each rank cuts its heads / columns out of every source
            qp = kp = gp = None
            if tp > 1:
                qp = slice(rank * hq * d, (rank + 1) * hq * d)
                kp = slice(kv0 * d, (kv0 + hkv) * d)
                gp = slice(rank * f, (rank + 1) * f)
            layer.qkv = _load_fused(snap, [f"{p}.self_attn.{x}_proj" for x in "qkv"], device, parts=[qp, kp, kp],
                                    name=f"{p}.self_attn.qkv_proj")
            layer.gate_up = _load_fused(snap, [f"{p}.mlp.gate_proj", f"{p}.mlp.up_proj"], device, parts=[gp, gp],
                                        interleave=True, name=f"{p}.mlp.gate_up_proj")
        layer.o = _load_lin(snap, f"{p}.self_attn.o_proj", device, cols=ocols)
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


def load_hybrid(full: Target, directory: str, device="cpu", tp: int = 1, rank: int = 0, seed: int = 0):
    """A hybrid-family model from a checkpoint directory: the published Nemotron-class tensor layout
    (weights/nemotron_layout.py), the published Qwen3.8-class layout (weights/qwen_layout.py), or this build's own
    snapshot (weights/snapshot.py: the model is built with this
    rank's geometry, then every tensor is overwritten with the stored one)."""
    from ..models.hybrid import HybridModel
    from . import snapshot
    index = Path(directory) / INDEX
    if index.exists() and "language_model.backbone.embeddings.weight" in json.loads(index.read_text())["weight_map"]:
        # the published Nemotron-class layout (one mixer per block, separate q / k / v and expert tensors)
        if tp != 1:
            raise NotImplementedError("the Nemotron-class checkpoint layout loads unsharded (tp = 1); save a per-rank "
                                      "snapshot of the loaded model for tensor-parallel serving")
        from . import nemotron_layout
        return nemotron_layout.load(full, directory, device, seed=seed)
    if index.exists():
        from . import qwen_layout
        if qwen_layout.is_layout(json.loads(index.read_text())["weight_map"]):
            # the published Qwen3.8-class layout (per-layer linear_attn / self_attn / mlp names)
            if tp != 1:
                raise NotImplementedError("the Qwen3.8-class checkpoint layout loads unsharded (tp = 1); save a "
                                          "per-rank snapshot of the loaded model for tensor-parallel serving")
            return qwen_layout.load(full, directory, device, seed=seed)
    model = HybridModel(full, device, seed=seed) if tp == 1 else HybridModel.sharded(full, tp, rank, device, seed=seed)
    snapshot.load_state(model, directory)
    return model
