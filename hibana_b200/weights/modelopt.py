"""ModelOpt-style quantised linear tensors in safetensors files.

NVFP4 linear `<name>`:  `<name>.weight` uint8 [N, K/2] (two e2m1 values per byte, low nibble first),
`<name>.weight_scale` float8_e4m3fn [N, K/16] (row-major, NOT swizzled), `<name>.weight_scale_2` fp32 scalar,
`<name>.input_scale` fp32 scalar (static activation scale).  FP8 linear: `<name>.weight` float8_e4m3fn [N, K],
`<name>.weight_scale` fp32 scalar, `<name>.input_scale` fp32 scalar.  On load the block scales are re-tiled into the
128x4 blocks the block-scaled MMA reads. Reference: hibana/weights/modelopt.py:89-184.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..models.linear import Linear
from ..ops import nvfp4
from ..ops.fp8 import Fp8Weight


def nvfp4_tensors(lin: Linear, name: str) -> dict:
    """The four checkpoint tensors of an NVFP4 linear (scales back in row-major order)."""
    assert lin.fmt == "nvfp4"
    w = lin.wq
    sf = nvfp4.unswizzle_sf(w.sf, w.rows, w.k // 16)
    return {f"{name}.weight": w.q.cpu().contiguous(), f"{name}.weight_scale": sf.cpu().view(torch.float8_e4m3fn),
            f"{name}.weight_scale_2": w.gscale.reshape(()).float().cpu(),
            f"{name}.input_scale": lin.input_scale.reshape(()).float().cpu()}


def load_nvfp4_linear(tensors: Mapping[str, torch.Tensor], name: str, device="cpu", rows=None, cols=None) -> Linear:
    """Builds a Linear from checkpoint tensors; `rows` / `cols` (slice or index tensor; cols in elements, multiple of
    16) cut a tensor-parallel shard out of the stored matrix without requantising."""
    q = tensors[f"{name}.weight"]
    sf = tensors[f"{name}.weight_scale"].view(torch.uint8)
    if rows is not None:
        q, sf = q[rows], sf[rows]
    if cols is not None:
        c0, c1 = cols.start or 0, cols.stop
        assert c0 % 16 == 0 and c1 % 16 == 0
        q, sf = q[:, c0 // 2:c1 // 2], sf[:, c0 // 16:c1 // 16]
    n, k = q.shape[0], q.shape[1] * 2
    gs = tensors[f"{name}.weight_scale_2"].reshape(1).float()
    wq = nvfp4.Nvfp4Tensor(q.contiguous().to(device), nvfp4.swizzle_sf(sf.contiguous()).to(device), gs.to(device), n, k)
    return Linear.from_nvfp4(wq, tensors[f"{name}.input_scale"].to(device), name=name)


def load_nvfp4_fused(tensors: Mapping[str, torch.Tensor], names: list, device="cpu", *, parts=None,
                      interleave: bool = False, cols=None, name: str = "") -> Linear:
    """One Linear out of several stored projections (q_proj + k_proj + v_proj, or gate_proj + up_proj), the way real
    ModelOpt / Hugging Face checkpoints ship them: rows are concatenated along N in the order of `names`
    (`interleave`: rows of the two sources alternate g0, u0, g1, u1 ..., what the SiLU-mul epilogue expects),
    `parts[i]` (slice or index tensor, may be None) first cuts this rank's rows out of source i. The sources must
    share one `weight_scale_2` (they were quantised as one matrix); the static activation scale is their largest
    `input_scale`. Nothing is requantised. Reference: hibana/weights/modelopt.py:108-184 (`load_nvfp4_linear(w, [q, k, v])`)."""
    qs, sfs, gss, ins = [], [], [], []
    for i, n in enumerate(names):
        q = tensors[f"{n}.weight"]
        sf = tensors[f"{n}.weight_scale"].view(torch.uint8)
        sel = parts[i] if parts is not None else None
        if sel is not None:
            q, sf = q[sel], sf[sel]
        if cols is not None:
            c0, c1 = cols.start or 0, cols.stop
            assert c0 % 16 == 0 and c1 % 16 == 0
            q, sf = q[:, c0 // 2:c1 // 2], sf[:, c0 // 16:c1 // 16]
        qs.append(q)
        sfs.append(sf)
        gss.append(float(tensors[f"{n}.weight_scale_2"].reshape(-1)[0]))
        ins.append(tensors[f"{n}.input_scale"].reshape(1).float())
    if any(abs(g - gss[0]) > 1e-12 * max(abs(gss[0]), 1e-30) for g in gss):
        raise ValueError(f"projections {names} do not share one weight_scale_2 ({gss}); they cannot be fused "
                         "without requantising")
    if interleave:
        assert len(qs) == 2 and qs[0].shape == qs[1].shape
        q = torch.stack((qs[0], qs[1]), dim=1).reshape(2 * qs[0].shape[0], qs[0].shape[1])
        sf = torch.stack((sfs[0], sfs[1]), dim=1).reshape(2 * sfs[0].shape[0], sfs[0].shape[1])
    else:
        q, sf = torch.cat(qs, 0), torch.cat(sfs, 0)
    n_rows, k = q.shape[0], q.shape[1] * 2
    gs = torch.tensor([gss[0]], dtype=torch.float32)
    wq = nvfp4.Nvfp4Tensor(q.contiguous().to(device), nvfp4.swizzle_sf(sf.contiguous()).to(device), gs.to(device),
                           n_rows, k)
    return Linear.from_nvfp4(wq, torch.stack(ins).max().reshape(1).to(device), name=name or names[0])


def fp8_tensors(w: Fp8Weight, input_scale: torch.Tensor, name: str) -> dict:
    return {f"{name}.weight": w.q.cpu(), f"{name}.weight_scale": w.scale.reshape(()).cpu(),
            f"{name}.input_scale": input_scale.reshape(()).float().cpu()}


def load_fp8_linear(tensors: Mapping[str, torch.Tensor], name: str, device="cpu") -> tuple[Fp8Weight, torch.Tensor]:
    return (Fp8Weight(tensors[f"{name}.weight"].to(device), tensors[f"{name}.weight_scale"].reshape(1).float().to(device)),
            tensors[f"{name}.input_scale"].reshape(1).float().to(device))


def unpack_fp4(q: torch.Tensor) -> torch.Tensor:
    """uint8 [.., K/2] -> fp32 e2m1 values [.., K]."""
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32,
                       device=q.device)
    lo, hi = lut[(q & 0xF).long()], lut[(q >> 4).long()]
    return torch.stack((lo, hi), dim=-1).flatten(-2)
