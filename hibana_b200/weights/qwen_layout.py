"""The Qwen3.8-class checkpoint layout: tensor names of the published hybrid checkpoint <-> this build's model.

The checkpoint names its tensors by decoder layer: `model.language_model.layers.{i}.input_layernorm`,
`.post_attention_layernorm`, one mixer per layer (`linear_attn.*` for a gated-delta-rule layer: `in_proj_qkv`,
`in_proj_z`, `in_proj_b`, `in_proj_a`, `conv1d.weight`, `A_log`, `dt_bias`, `norm.weight`, `out_proj`;
`self_attn.*` for a gated full-attention layer: `q_proj` with rows [head: q | gate], `k_proj`, `v_proj`, `o_proj`,
`q_norm`, `k_norm`) and a dense MLP (`mlp.gate_proj|up_proj|down_proj`), plus `embed_tokens`, `norm`, `lm_head` and
the multi-token-prediction head under `mtp.` (`fc`, `pre_fc_norm_embedding`, `pre_fc_norm_hidden`, `layers.0.*`,
`norm`). A projection is stored in one of three forms:

* ModelOpt NVFP4 (`weight` two codes per byte, `weight_scale`, `weight_scale_2`, `input_scale`): taken as stored,
  fused projections concatenate (or pair-interleave, gate / up) their rows; nothing is requantised;
* FP8 with one scale per 128 x 128 block (`weight` e4m3, `weight_scale_inv` fp32): expanded to bf16 and served as a
  bf16 projection (exact to the stored values up to bf16 rounding of value x scale), or rounded to the target's
  format with `requantize=True`;
* plain bf16.

`save` writes a model back under the same names (fixtures, exporting); with `fp8_mixers` the mixer projections are
written in the block-scaled FP8 form.
Reference: hibana/model/qwen38.py:31-123, gdn.py:63-76, attention.py:33-39, mlp.py:18-21, mtp.py:20-44.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from ..models.linear import Linear, interleave_pairs
from ..target import GATED_ATTN, GDN, MLP, Target
from .checkpoint import INDEX, Snapshot, _lin_tensors, _load_fused, _load_lin, _split_rows

PREFIX = "model.language_model"
MTP = "mtp"
FP8_BLOCK = 128


# ---- block-scaled FP8
def fp8_block_dequant(w: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """[rows, cols] e4m3 x one fp32 scale per 128 x 128 block -> bf16."""
    rows, cols = w.shape
    s = scale_inv.float().repeat_interleave(FP8_BLOCK, 0)[:rows].repeat_interleave(FP8_BLOCK, 1)[:, :cols]
    return (w.float() * s).to(torch.bfloat16)


def fp8_block_quant(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, cols] -> (e4m3 values, fp32 scale per 128 x 128 block): block maximum maps to 448."""
    rows, cols = w.shape
    rb, cb = -(-rows // FP8_BLOCK), -(-cols // FP8_BLOCK)
    pad = torch.zeros(rb * FP8_BLOCK, cb * FP8_BLOCK, dtype=torch.float32)
    pad[:rows, :cols] = w.float()
    amax = pad.view(rb, FP8_BLOCK, cb, FP8_BLOCK).abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (pad.view(rb, FP8_BLOCK, cb, FP8_BLOCK) / scale[:, None, :, None]).reshape(rb * FP8_BLOCK, cb * FP8_BLOCK)
    return q[:rows, :cols].to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def _bf16_source(snap: Snapshot, name: str) -> torch.Tensor:
    w = snap[f"{name}.weight"]
    if f"{name}.weight_scale_inv" in snap:
        return fp8_block_dequant(w, snap[f"{name}.weight_scale_inv"])
    return w.to(torch.bfloat16)


def _projection(snap: Snapshot, names: list, device, *, interleave: bool = False, name: str = "", fmt: str = "bf16"):
    """One `Linear` from one or several stored projections, whichever form they are stored in."""
    if f"{names[0]}.weight_scale" in snap:
        if len(names) == 1:
            return _load_lin(snap, names[0], device)
        return _load_fused(snap, names, device, interleave=interleave, name=name)
    ws = [_bf16_source(snap, n) for n in names]
    w = interleave_pairs(ws[0], ws[1]) if interleave else torch.cat(ws, 0)
    return Linear(w.contiguous(), fmt, name=name or names[0]).to(device)


def _proj_tensors(lin: Linear, name: str, fp8: bool) -> dict:
    if fp8 and lin.fmt == "bf16":
        q, s = fp8_block_quant(lin.weight.cpu())
        return {f"{name}.weight": q, f"{name}.weight_scale_inv": s}
    return _lin_tensors(lin, name)


def _split_tensors(lin: Linear, name_rows: list, fp8: bool, deinterleave: bool = False) -> dict:
    if fp8 and lin.fmt == "bf16":
        out = {}
        for name, sel in name_rows:
            q, s = fp8_block_quant(lin.weight.cpu()[sel])
            out[f"{name}.weight"], out[f"{name}.weight_scale_inv"] = q, s
        return out
    return _split_rows(lin, name_rows, deinterleave=deinterleave)


# ---- one sublayer <-> its names
def _gdn_tensors(sub, p: str, t: Target, fp8: bool) -> dict:
    qk, vd = t.gdn_k_heads * t.gdn_head_dim, t.gdn_v_heads * t.gdn_head_dim
    out = _split_tensors(sub.in_qkvz, [(f"{p}.in_proj_qkv", slice(0, 2 * qk + vd)),
                                       (f"{p}.in_proj_z", slice(2 * qk + vd, 2 * qk + 2 * vd))], fp8)
    ba = sub.in_ba.weight.cpu()
    out[f"{p}.in_proj_b.weight"], out[f"{p}.in_proj_a.weight"] = ba[:t.gdn_v_heads], ba[t.gdn_v_heads:]
    out[f"{p}.conv1d.weight"] = sub.conv_w.cpu().unsqueeze(1)
    out[f"{p}.A_log"], out[f"{p}.dt_bias"] = sub.a_log.cpu(), sub.dt_bias.cpu()
    out[f"{p}.norm.weight"] = sub.norm_w.cpu()
    out.update(_proj_tensors(sub.out_proj, f"{p}.out_proj", fp8))
    return out


def _load_gdn(sub, snap: Snapshot, p: str, t: Target, dev, fmt: str, name: str) -> None:
    sub.in_qkvz = _projection(snap, [f"{p}.in_proj_qkv", f"{p}.in_proj_z"], dev, name=name + ".in_qkvz", fmt=fmt)
    ba = torch.cat([snap[f"{p}.in_proj_b.weight"], snap[f"{p}.in_proj_a.weight"]], 0).to(torch.bfloat16)
    sub.in_ba = Linear(ba.contiguous(), "bf16", name=name + ".in_ba").to(dev)
    sub.conv_w = snap[f"{p}.conv1d.weight"].reshape(-1, t.conv_width).to(torch.bfloat16).to(dev).contiguous()
    sub.a_log, sub.dt_bias = snap[f"{p}.A_log"].float().to(dev), snap[f"{p}.dt_bias"].float().to(dev)
    sub.norm_w = snap[f"{p}.norm.weight"].to(sub.norm_w.dtype).to(dev)
    sub.norm_w_heads, sub._norm_w_key = None, None
    sub.out_proj = _projection(snap, [f"{p}.out_proj"], dev, name=name + ".out_proj", fmt=fmt)
    sub.first = sub.in_qkvz
    want = 2 * t.gdn_k_heads * t.gdn_head_dim + 2 * t.gdn_v_heads * t.gdn_head_dim
    if sub.in_qkvz.out_features != want:
        raise ValueError(f"{p}: in_proj_qkv + in_proj_z have {sub.in_qkvz.out_features} rows, the target wants {want}")


def _attn_tensors(sub, p: str, t: Target, fp8: bool) -> dict:
    d = t.head_dim
    nq, nk = t.q_heads * d * (2 if sub.gated else 1), t.kv_heads * d
    out = _split_tensors(sub.qkv, [(f"{p}.q_proj", slice(0, nq)), (f"{p}.k_proj", slice(nq, nq + nk)),
                                   (f"{p}.v_proj", slice(nq + nk, nq + 2 * nk))], fp8)
    out.update(_proj_tensors(sub.o, f"{p}.o_proj", fp8))
    if sub.q_norm is not None:
        out[f"{p}.q_norm.weight"], out[f"{p}.k_norm.weight"] = sub.q_norm.cpu(), sub.k_norm.cpu()
    return out


def _load_attn(sub, snap: Snapshot, p: str, t: Target, dev, fmt: str, name: str) -> None:
    sub.qkv = _projection(snap, [f"{p}.q_proj", f"{p}.k_proj", f"{p}.v_proj"], dev, name=name + ".qkv", fmt=fmt)
    sub.o = _projection(snap, [f"{p}.o_proj"], dev, name=name + ".o", fmt=fmt)
    if sub.q_norm is not None:
        sub.q_norm = snap[f"{p}.q_norm.weight"].to(sub.q_norm.dtype).to(dev)
        sub.k_norm = snap[f"{p}.k_norm.weight"].to(sub.k_norm.dtype).to(dev)
    sub.first = sub.qkv
    want = (t.q_heads * (2 if sub.gated else 1) + 2 * t.kv_heads) * t.head_dim
    if sub.qkv.out_features != want:
        raise ValueError(f"{p}: q / k / v have {sub.qkv.out_features} rows together, the target wants {want} "
                         f"({'gated' if sub.gated else 'plain'} attention)")


def _mlp_tensors(sub, p: str) -> dict:
    n = sub.up.out_features
    out = _split_rows(sub.up, [(f"{p}.gate_proj", slice(0, n, 2)), (f"{p}.up_proj", slice(1, n, 2))])
    out.update(_lin_tensors(sub.down, f"{p}.down_proj"))
    return out


def _load_mlp(sub, snap: Snapshot, p: str, dev, fmt: str, name: str) -> None:
    sub.up = _projection(snap, [f"{p}.gate_proj", f"{p}.up_proj"], dev, interleave=True, name=name + ".gate_up", fmt=fmt)
    sub.down = _projection(snap, [f"{p}.down_proj"], dev, name=name + ".down", fmt=fmt)
    sub.first = sub.up


# ---- whole model
def tensors_of(model, fp8_mixers: bool = False) -> dict:
    """Every tensor of a tensor-parallel-free Qwen3.8-class model under the checkpoint's names."""
    t = model.target
    out = {f"{PREFIX}.embed_tokens.weight": model.embed.cpu(), f"{PREFIX}.norm.weight": model.final_norm.cpu()}
    if model.lm_head is not model.embed:
        out["lm_head.weight"] = model.lm_head.cpu()
    for i, blk in enumerate(model.blocks):
        p = f"{PREFIX}.layers.{i}"
        mixer, ffn = t.layers[i]
        if ffn != MLP or mixer not in (GDN, GATED_ATTN):
            raise ValueError(f"block {i}: the layout has a gated-delta-rule or gated-attention mixer and a dense MLP "
                             f"per layer, this block is {mixer!r} + {ffn!r}")
        out[f"{p}.input_layernorm.weight"] = blk.mixer_norm.cpu()
        out[f"{p}.post_attention_layernorm.weight"] = blk.ffn_norm.cpu()
        if mixer == GDN:
            out.update(_gdn_tensors(blk.mixer, f"{p}.linear_attn", t, fp8_mixers))
        else:
            out.update(_attn_tensors(blk.mixer, f"{p}.self_attn", t, fp8_mixers))
        out.update(_mlp_tensors(blk.ffn, f"{p}.mlp"))
    h = getattr(model, "mtp", None)
    if h is not None:
        out[f"{MTP}.fc.weight"] = h.fc.weight.cpu()
        out[f"{MTP}.pre_fc_norm_embedding.weight"], out[f"{MTP}.pre_fc_norm_hidden.weight"] = h.enorm.cpu(), h.hnorm.cpu()
        out[f"{MTP}.layers.0.input_layernorm.weight"] = h.attn_norm.cpu()
        out[f"{MTP}.layers.0.post_attention_layernorm.weight"] = h.mlp_norm.cpu()
        out[f"{MTP}.norm.weight"] = h.final_norm.cpu()
        out.update(_attn_tensors(h.attn, f"{MTP}.layers.0.self_attn", t, False))
        out.update(_mlp_tensors(h.mlp, f"{MTP}.layers.0.mlp"))
    return {k: v.contiguous().clone() for k, v in out.items()}     # (no two names may share storage in a file)


def save(model, directory, layers_per_file: int = 8, fp8_mixers: bool = False) -> Path:
    """Writes `model` (tp = 1) as safetensors shards + index under the checkpoint's names."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    tensors = tensors_of(model, fp8_mixers)

    def shard_of(name: str) -> int:
        return 1 + int(name.split(".")[3]) // layers_per_file if name.startswith(f"{PREFIX}.layers.") else 0
    groups: dict = {}
    for name, ten in tensors.items():
        groups.setdefault(shard_of(name), {})[name] = ten
    index = {}
    for i, (_, group) in enumerate(sorted(groups.items())):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(group, str(d / fname))
        index.update({name: fname for name in group})
    (d / INDEX).write_text(json.dumps({"metadata": {"layout": "qwen38"}, "weight_map": index}, indent=1))
    return d


def is_layout(weight_map: dict) -> bool:
    return f"{PREFIX}.embed_tokens.weight" in weight_map and any(".linear_attn." in k for k in weight_map)


def load(target: Target, directory, device="cpu", seed: int = 0, requantize: bool = False):
    """A `HybridModel` of `target` with every tensor taken from the checkpoint directory (tp = 1). Projections stored
    as block-scaled FP8 or bf16 are served in bf16 unless `requantize` rounds them to the target's weight format."""
    from ..models.hybrid import HybridModel
    snap = Snapshot(str(directory))
    model = HybridModel(target, device, seed=seed)
    dev, t = model.device, target
    fmt = t.weight_format if requantize else "bf16"
    model.embed = snap[f"{PREFIX}.embed_tokens.weight"].to(torch.bfloat16).to(dev)
    model.final_norm = snap[f"{PREFIX}.norm.weight"].to(model.final_norm.dtype).to(dev)
    if "lm_head.weight" in snap:
        if "lm_head.weight_scale" in snap:        # an NVFP4 head: this build's head is a bf16 matrix
            model.lm_head = _load_lin(snap, "lm_head", "cpu").dequantized().to(torch.bfloat16).to(dev)
        else:
            model.lm_head = snap["lm_head.weight"].to(torch.bfloat16).to(dev)
    else:
        model.lm_head = model.embed
    for i, blk in enumerate(model.blocks):
        p = f"{PREFIX}.layers.{i}"
        mixer, ffn = t.layers[i]
        if ffn != MLP or mixer not in (GDN, GATED_ATTN):
            raise ValueError(f"block {i}: no checkpoint names for {mixer!r} + {ffn!r}")
        blk.mixer_norm = snap[f"{p}.input_layernorm.weight"].to(blk.mixer_norm.dtype).to(dev)
        blk.ffn_norm = snap[f"{p}.post_attention_layernorm.weight"].to(blk.ffn_norm.dtype).to(dev)
        if mixer == GDN:
            _load_gdn(blk.mixer, snap, f"{p}.linear_attn", t, dev, fmt, f"l{i}.mixer")
        else:
            _load_attn(blk.mixer, snap, f"{p}.self_attn", t, dev, fmt, f"l{i}.mixer")
        _load_mlp(blk.ffn, snap, f"{p}.mlp", dev, fmt, f"l{i}.ffn")
    h = getattr(model, "mtp", None)
    if h is not None and f"{MTP}.fc.weight" in snap:
        h.fc = Linear(snap[f"{MTP}.fc.weight"].to(torch.bfloat16), "bf16", name="mtp.fc").to(dev)
        h.enorm = snap[f"{MTP}.pre_fc_norm_embedding.weight"].to(h.enorm.dtype).to(dev)
        h.hnorm = snap[f"{MTP}.pre_fc_norm_hidden.weight"].to(h.hnorm.dtype).to(dev)
        h.attn_norm = snap[f"{MTP}.layers.0.input_layernorm.weight"].to(h.attn_norm.dtype).to(dev)
        h.mlp_norm = snap[f"{MTP}.layers.0.post_attention_layernorm.weight"].to(h.mlp_norm.dtype).to(dev)
        h.final_norm = snap[f"{MTP}.norm.weight"].to(h.final_norm.dtype).to(dev)
        _load_attn(h.attn, snap, f"{MTP}.layers.0.self_attn", t, dev, fmt, "mtp.attn")
        _load_mlp(h.mlp, snap, f"{MTP}.layers.0.mlp", dev, fmt, "mtp.mlp")
    return model
