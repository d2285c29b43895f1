"""The Nemotron-class checkpoint layout: tensor names of the published NVFP4 checkpoint <-> this build's model.

A Nemotron-class (and Bolt-class) checkpoint names its tensors by block: `language_model.backbone.layers.{i}.norm`,
`.mixer.*` with one mixer per block (Mamba-2: `in_proj`, `out_proj`, `conv1d.weight|bias`, `A_log`, `D`, `dt_bias`,
`norm.weight`; attention: `q_proj`, `k_proj`, `v_proj`, `o_proj`; latent MoE: `gate.weight`,
`gate.e_score_correction_bias`, `fc1_latent_proj`, `fc2_latent_proj`, `shared_experts.up_proj|down_proj`,
`experts.{e}.up_proj|down_proj`), plus `backbone.embeddings`, `backbone.norm_f` and `lm_head`. NVFP4 projections are
the four ModelOpt tensors (`weight` two codes per byte, `weight_scale` e4m3 per 16 columns in row-major order,
`weight_scale_2`, `input_scale`). `load` builds this build's `HybridModel` from such a directory without
requantising anything: q / k / v are fused by concatenating rows (they must share one `weight_scale_2`), the routed
experts are stacked with their own per-expert scales, block scales are re-tiled into the tensor core's 128 x 4
layout. `save` writes a model back under the same names (fixtures, and exporting a calibrated model).
Reference: hibana/model/nemotron/model.py:40,77-83,142,171-172, mamba.py:28-33, attention.py:34-36, moe.py:327-375.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from ..models.linear import Linear
from ..ops import moe as moe_ops
from ..ops import nvfp4
from ..target import ATTN, GATED_ATTN, LATENT_MOE, MAMBA2, MOE, Target
from . import modelopt
from .checkpoint import INDEX, Snapshot, _lin_tensors, _load_fused, _load_lin, _split_rows

PREFIX = "language_model"
BACKBONE = f"{PREFIX}.backbone"


def _expert_tensors(ew: moe_ops.ExpertWeights, which: int, e: int, name: str) -> dict:
    """Checkpoint tensors of expert `e`'s fc1 (which = 1) or fc2 matrix."""
    w = ew.fc1 if which == 1 else ew.fc2
    rows = ew.n1 if which == 1 else (w.rows if ew.fmt == "nvfp4" else w.shape[0]) // ew.experts
    sel = slice(e * rows, (e + 1) * rows)
    if ew.fmt == "bf16":
        return {f"{name}.weight": w[sel].cpu().contiguous()}
    sf = nvfp4.unswizzle_sf(w.sf, w.rows, w.k // 16)
    in_scale = ew.fc1_in_scale if which == 1 else ew.fc2_in_scale
    return {f"{name}.weight": w.q[sel].cpu().contiguous(),
            f"{name}.weight_scale": sf[sel].cpu().contiguous().view(torch.float8_e4m3fn),
            f"{name}.weight_scale_2": w.gscale[e].reshape(()).float().cpu(),
            f"{name}.input_scale": in_scale.reshape(()).float().cpu()}


def tensors_of(model) -> dict:
    """Every tensor of a tensor-parallel-free hybrid model under the checkpoint's names."""
    t = model.target
    out = {f"{BACKBONE}.embeddings.weight": model.embed.cpu(), f"{BACKBONE}.norm_f.weight": model.final_norm.cpu(),
           f"{PREFIX}.lm_head.weight": model.lm_head.cpu()}
    for i, blk in enumerate(model.blocks):
        p = f"{BACKBONE}.layers.{i}"
        subs = [(n, s) for n, s in blk.sublayers() if s is not None]
        if len(subs) != 1:
            raise ValueError(f"block {i}: the layout has one mixer per block, this block has {len(subs)} sublayers")
        norm, sub = subs[0]
        out[f"{p}.norm.weight"] = norm.cpu()
        m = f"{p}.mixer"
        kind = t.layers[i][0] if blk.mixer is not None else t.layers[i][1]
        if kind == MAMBA2:
            out.update(_lin_tensors(sub.in_proj, f"{m}.in_proj"))
            out.update(_lin_tensors(sub.out_proj, f"{m}.out_proj"))
            out[f"{m}.conv1d.weight"] = sub.conv_w.cpu().unsqueeze(1).contiguous()
            out[f"{m}.conv1d.bias"] = sub.conv_b.cpu()
            out[f"{m}.A_log"], out[f"{m}.D"] = sub.a_log.cpu(), sub.d_skip.cpu()
            out[f"{m}.dt_bias"], out[f"{m}.norm.weight"] = sub.dt_bias.cpu(), sub.norm_w.cpu()
        elif kind in (ATTN, GATED_ATTN):
            hd = t.head_dim
            nq = t.q_heads * hd * (2 if kind == GATED_ATTN else 1)
            nk = t.kv_heads * hd
            out.update(_split_rows(sub.qkv, [(f"{m}.q_proj", slice(0, nq)), (f"{m}.k_proj", slice(nq, nq + nk)),
                                             (f"{m}.v_proj", slice(nq + nk, nq + 2 * nk))]))
            out.update(_lin_tensors(sub.o, f"{m}.o_proj"))
        elif kind in (MOE, LATENT_MOE):
            out[f"{m}.gate.weight"] = sub.router.weight.cpu()
            if sub.sel_bias is not None:
                out[f"{m}.gate.e_score_correction_bias"] = sub.sel_bias.cpu()
            if sub.fc1_latent is not None:
                out[f"{m}.fc1_latent_proj.weight"] = sub.fc1_latent.weight.cpu()
                out[f"{m}.fc2_latent_proj.weight"] = sub.fc2_latent.weight.cpu()
            if sub.shared is not None:
                out.update(_lin_tensors(sub.shared.up, f"{m}.shared_experts.up_proj"))
                out.update(_lin_tensors(sub.shared.down, f"{m}.shared_experts.down_proj"))
            ew = sub.experts
            for e in range(ew.experts):
                out.update(_expert_tensors(ew, 1, e, f"{m}.experts.{e}.up_proj"))
                out.update(_expert_tensors(ew, 2, e, f"{m}.experts.{e}.down_proj"))
        else:
            raise ValueError(f"block {i}: no checkpoint names for a {kind!r} sublayer")
    return {k: v.contiguous().clone() for k, v in out.items()}     # (no two names may share storage in a file)


def save(model, directory, blocks_per_file: int = 8) -> Path:
    """Writes `model` (tp = 1) as safetensors shards + index under the checkpoint's names."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    tensors = tensors_of(model)

    def shard_of(name: str) -> int:
        parts = name.split(".")
        return 1 + int(parts[3]) // blocks_per_file if name.startswith(f"{BACKBONE}.layers.") else 0
    groups: dict = {}
    for name, ten in tensors.items():
        groups.setdefault(shard_of(name), {})[name] = ten
    index = {}
    for i, (_, group) in enumerate(sorted(groups.items())):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(group, str(d / fname))
        index.update({name: fname for name in group})
    (d / INDEX).write_text(json.dumps({"metadata": {"format": "modelopt-nvfp4", "layout": "nemotron"},
                                       "weight_map": index}, indent=1))
    return d


def _load_experts(snap: Snapshot, prefix: str, t: Target, device) -> moe_ops.ExpertWeights:
    """The routed experts of one layer, stacked, with their stored codes and scales."""
    names1 = [f"{prefix}.experts.{e}.up_proj" for e in range(t.experts)]
    names2 = [f"{prefix}.experts.{e}.down_proj" for e in range(t.experts)]
    width = t.latent or t.hidden
    if f"{names1[0]}.weight_scale" not in snap:
        fc1 = torch.stack([snap[f"{n}.weight"] for n in names1])
        fc2 = torch.stack([snap[f"{n}.weight"] for n in names2])
        return moe_ops.ExpertWeights.create(fc1, fc2, t.moe_act, "bf16").to(device)

    def stack(names):
        q = torch.cat([snap[f"{n}.weight"] for n in names], 0)
        sf = torch.cat([snap[f"{n}.weight_scale"].view(torch.uint8) for n in names], 0)
        gs = torch.stack([snap[f"{n}.weight_scale_2"].reshape(()).float() for n in names])
        ins = torch.stack([snap[f"{n}.input_scale"].reshape(()).float() for n in names]).max().reshape(1)
        return nvfp4.Nvfp4Tensor(q.contiguous(), nvfp4.swizzle_sf(sf.contiguous()), gs, q.shape[0], q.shape[1] * 2), gs, ins
    q1, g1, s1 = stack(names1)
    q2, g2, s2 = stack(names2)
    inter = q2.k
    if q1.k != width:
        raise ValueError(f"{prefix}: expert input width {q1.k} != {width}")
    return moe_ops.ExpertWeights(t.experts, width, inter, t.moe_act, "nvfp4", q1, q2, (g1 * s1).contiguous(),
                                 (g2 * s2).contiguous(), s1, s2).to(device)


def load(target: Target, directory, device="cpu", seed: int = 0):
    """A `HybridModel` of `target` with every tensor taken from the checkpoint directory (tp = 1)."""
    from ..models.hybrid import HybridModel
    snap = Snapshot(str(directory))
    model = HybridModel(target, device, seed=seed)
    dev = model.device
    t = target
    model.embed = snap[f"{BACKBONE}.embeddings.weight"].to(torch.bfloat16).to(dev)
    model.final_norm = snap[f"{BACKBONE}.norm_f.weight"].to(model.final_norm.dtype).to(dev)
    model.lm_head = snap[f"{PREFIX}.lm_head.weight"].to(torch.bfloat16).to(dev) if f"{PREFIX}.lm_head.weight" in snap \
        else model.embed
    for i, blk in enumerate(model.blocks):
        p = f"{BACKBONE}.layers.{i}"
        m = f"{p}.mixer"
        norm = snap[f"{p}.norm.weight"]
        if blk.mixer is not None:
            blk.mixer_norm = norm.to(blk.mixer_norm.dtype).to(dev)
            sub, kind = blk.mixer, t.layers[i][0]
        else:
            blk.ffn_norm = norm.to(blk.ffn_norm.dtype).to(dev)
            sub, kind = blk.ffn, t.layers[i][1]
        if kind == MAMBA2:
            sub.in_proj = _load_lin(snap, f"{m}.in_proj", dev)
            sub.out_proj = _load_lin(snap, f"{m}.out_proj", dev)
            sub.conv_w = snap[f"{m}.conv1d.weight"].reshape(-1, t.conv_width).to(torch.bfloat16).to(dev).contiguous()
            sub.conv_b = snap[f"{m}.conv1d.bias"].to(torch.bfloat16).to(dev)
            sub.a_log, sub.d_skip = snap[f"{m}.A_log"].float().to(dev), snap[f"{m}.D"].float().to(dev)
            sub.dt_bias = snap[f"{m}.dt_bias"].float().to(dev)
            sub.norm_w = snap[f"{m}.norm.weight"].to(sub.norm_w.dtype).to(dev)
            sub.first = sub.in_proj
            if hasattr(sub, "norm_w_heads"):
                sub.norm_w_heads = None          # derived cache of the gated norm: rebuilt on first use
        elif kind in (ATTN, GATED_ATTN):
            sub.qkv = _load_fused(snap, [f"{m}.q_proj", f"{m}.k_proj", f"{m}.v_proj"], dev, name=f"l{i}.mixer.qkv")
            sub.o = _load_lin(snap, f"{m}.o_proj", dev)
            sub.first = sub.qkv
        elif kind in (MOE, LATENT_MOE):
            sub.router = Linear(snap[f"{m}.gate.weight"], "bf16", name=f"l{i}.ffn.router").to(dev)
            if f"{m}.gate.e_score_correction_bias" in snap:
                sub.sel_bias = snap[f"{m}.gate.e_score_correction_bias"].float().to(dev)
            if sub.fc1_latent is not None:
                sub.fc1_latent = Linear(snap[f"{m}.fc1_latent_proj.weight"], "bf16", name=f"l{i}.ffn.fc1_latent").to(dev)
                sub.fc2_latent = Linear(snap[f"{m}.fc2_latent_proj.weight"], "bf16", name=f"l{i}.ffn.fc2_latent").to(dev)
            if sub.shared is not None:
                sub.shared.up = _load_lin(snap, f"{m}.shared_experts.up_proj", dev)
                sub.shared.down = _load_lin(snap, f"{m}.shared_experts.down_proj", dev)
                sub.shared.first = sub.shared.up
            sub.experts = _load_experts(snap, m, t.block(i), dev)
        else:
            raise ValueError(f"block {i}: no checkpoint names for a {kind!r} sublayer")
    return model
