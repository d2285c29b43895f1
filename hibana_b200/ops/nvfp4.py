"""NVFP4 format helpers and activation quantisers.

Format (ModelOpt NVFP4, as loaded by the reference in hibana/weights/modelopt.py:130-184): e2m1 values packed
two per byte (low nibble first), one e4m3 scale per 16 elements along K, and an fp32 per-tensor scale, so
``x ~= e2m1 * e4m3_scale * global_scale``. Block scales are kept in the 128x4 "swizzled" layout the tensor
cores consume: 512-byte blocks covering 128 rows x 4 scales, byte ``(r % 32) * 16 + (r // 32) * 4 + j``.

The torch functions here are the fp32 reference of the CUDA quantisers in csrc/quant.cu and are what runs on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as nv

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# Rounding boundaries between neighbouring e2m1 magnitudes; a tie goes to the code with an even mantissa.
_BOUNDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_TIE_UP = (False, True, False, True, False, True, False)


def k_atoms(k: int) -> int:
    """Number of 64-element K atoms of a scale tensor, padded to a whole 256-element K tile."""
    return ((k + 255) // 256) * 4


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """4-bit codes (sign in bit 3) of values already divided by their block scale."""
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.int32)
    for b, up in zip(_BOUNDS, _TIE_UP):
        code += (a >= b).int() if up else (a > b).int()
    return code | ((x < 0).int() << 3)


def e2m1_values(codes: torch.Tensor) -> torch.Tensor:
    mag = E2M1.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 bytes (uint8), saturating."""
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def from_e4m3(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).float()


def swizzle_sf(sf: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] uint8 row-major scales -> [ceil(rows/128), k_atoms, 512] swizzled blocks (zero padded)."""
    rows, groups = sf.shape
    ka = k_atoms(groups * 16)
    rb = (rows + 127) // 128
    rb += rb & 1 if rb > 1 else 0  # whole 256-row tiles, so a 128 x 256 MMA tile never reads past the end
    full = torch.zeros(rb * 128, ka * 4, dtype=torch.uint8, device=sf.device)
    full[:rows, :groups] = sf
    # [rb, 4 (r // 32), 32 (r % 32), ka, 4 (j)] -> [rb, ka, 32, 4, 4]
    v = full.view(rb, 4, 32, ka, 4).permute(0, 3, 2, 1, 4).contiguous()
    return v.view(rb, ka, 512)


def unswizzle_sf(blocks: torch.Tensor, rows: int, groups: int) -> torch.Tensor:
    rb, ka, _ = blocks.shape
    v = blocks.view(rb, ka, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(rb * 128, ka * 4)
    return v[:rows, :groups].contiguous()


def quantize_ref(x: torch.Tensor, global_scale: float | torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Reference quantiser. x [M, K] -> (packed uint8 [M, K/2], row-major scale bytes uint8 [M, K/16])."""
    m, k = x.shape
    assert k % 16 == 0
    gs = float(global_scale)
    xf = x.float().view(m, k // 16, 16)
    amax = xf.abs().amax(dim=-1)
    sfb = to_e4m3(amax * (1.0 / 6.0) * (1.0 / gs))
    sf = from_e4m3(sfb)
    inv = torch.where(sf > 0, 1.0 / (sf * gs), torch.zeros_like(sf))
    codes = e2m1_codes(xf * inv.unsqueeze(-1)).view(m, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
    return packed, sfb


def dequantize_ref(packed: torch.Tensor, sfb: torch.Tensor, global_scale: float | torch.Tensor) -> torch.Tensor:
    """(packed [M, K/2], scale bytes [M, K/16]) -> fp32 [M, K]."""
    m, kh = packed.shape
    p = packed.int()
    codes = torch.stack((p & 15, p >> 4), dim=-1).view(m, kh * 2)
    vals = e2m1_values(codes).view(m, kh * 2 // 16, 16)
    return (vals * from_e4m3(sfb).unsqueeze(-1)).view(m, kh * 2) * float(global_scale)


@dataclass
class Nvfp4Tensor:
    """A quantised [rows, k] matrix: packed values, swizzled scale blocks and the per-tensor scale (device)."""

    q: torch.Tensor          # uint8 [rows, k/2]
    sf: torch.Tensor         # uint8 [ceil(rows/128), k_atoms, 512]
    gscale: torch.Tensor     # fp32 scalar tensor
    rows: int
    k: int

    @property
    def ka(self) -> int:
        return self.sf.shape[1]

    def dequantize(self) -> torch.Tensor:
        sfb = unswizzle_sf(self.sf, self.rows, self.k // 16)
        return dequantize_ref(self.q, sfb, self.gscale)


def quantize_weight(w: torch.Tensor, global_scale: Optional[float] = None) -> Nvfp4Tensor:
    """Quantises a weight matrix [N, K] (any float dtype) the way ModelOpt does: global = amax / (6 * 448)."""
    if global_scale is None:
        global_scale = max(float(w.abs().max()) / (6.0 * 448.0), 1e-12)
    if w.is_cuda and nv.available():
        # Large matrices: the device quantiser (same arithmetic on the bf16-rounded weights).
        gs = torch.tensor(global_scale, dtype=torch.float32, device=w.device)
        t = quantize(w.to(torch.bfloat16).contiguous(), gs)
        return Nvfp4Tensor(t.q, t.sf, gs, w.shape[0], w.shape[1])
    wf = w.float()
    packed, sfb = quantize_ref(wf, global_scale)
    return Nvfp4Tensor(packed, swizzle_sf(sfb), torch.tensor(global_scale, dtype=torch.float32, device=w.device),
                       w.shape[0], w.shape[1])


nv.register("hb_quant_nvfp4", [nv.P, nv.L, nv.I, nv.I, nv.I, nv.P, nv.P, nv.P, nv.I, nv.P])
nv.register("hb_norm_quant_nvfp4", [nv.P, nv.P, nv.P, nv.F, nv.I, nv.I, nv.I, nv.I, nv.P, nv.P, nv.P, nv.P, nv.P])

MODE_PLAIN, MODE_SILU_SPLIT, MODE_SILU_PAIRS = 0, 1, 2


def _alloc(m: int, k: int, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    ka = k_atoms(k)
    q = torch.empty(m, k // 2, dtype=torch.uint8, device=device)
    rb = (m + 127) // 128
    rb += rb & 1 if rb > 1 else 0
    sf = torch.empty(rb, ka, 512, dtype=torch.uint8, device=device)
    return q, sf


def _silu_mul(x: torch.Tensor, mode: int) -> torch.Tensor:
    if mode == MODE_SILU_SPLIT:
        g, u = x.float().chunk(2, dim=-1)
    else:
        g, u = x.float()[:, 0::2], x.float()[:, 1::2]
    return (torch.nn.functional.silu(g) * u).to(x.dtype)


def quantize(x: torch.Tensor, gscale: torch.Tensor, mode: int = MODE_PLAIN) -> Nvfp4Tensor:
    """bf16 activations [M, K] -> NVFP4 with the static per-tensor scale `gscale` (fp32 scalar tensor).

    mode SILU_SPLIT / SILU_PAIRS first applies silu(gate) * up on a [M, 2K] input (gate|up halves, or
    gate/up interleaved pairwise) in the same pass.
    """
    m = x.shape[0]
    k = x.shape[1] if mode == MODE_PLAIN else x.shape[1] // 2
    if nv.use_native(x):
        assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
        q, sf = _alloc(m, k, x.device)
        nv.check(nv.lib().hb_quant_nvfp4(x.data_ptr(), x.stride(0), m, k, sf.shape[1], gscale.data_ptr(),
                                         q.data_ptr(), sf.data_ptr(), mode, nv.stream()), "hb_quant_nvfp4")
        return Nvfp4Tensor(q, sf, gscale, m, k)
    y = x if mode == MODE_PLAIN else _silu_mul(x, mode)
    packed, sfb = quantize_ref(y, gscale)
    return Nvfp4Tensor(packed, swizzle_sf(sfb), gscale, m, k)


def rmsnorm_quantize(x: torch.Tensor, weight: torch.Tensor, eps: float, gscale: torch.Tensor,
                     residual: Optional[torch.Tensor] = None, gemma: bool = False,
                     want_normed: bool = False) -> tuple[Nvfp4Tensor, Optional[torch.Tensor]]:
    """(residual += x;) y = rmsnorm(residual or x) * w -> NVFP4 in one pass. `residual` is updated in place.

    Returns (quantised y, y in bf16 if want_normed).
    """
    m, k = x.shape
    if nv.use_native(x):
        q, sf = _alloc(m, k, x.device)
        normed = torch.empty_like(x) if want_normed else None
        nv.check(nv.lib().hb_norm_quant_nvfp4(x.data_ptr(), nv.ptr(residual), weight.data_ptr(), eps, int(gemma), m, k,
                                              sf.shape[1], gscale.data_ptr(), q.data_ptr(), sf.data_ptr(),
                                              nv.ptr(normed), nv.stream()), "hb_norm_quant_nvfp4")
        return Nvfp4Tensor(q, sf, gscale, m, k), normed
    h = x
    if residual is not None:
        residual.copy_((x.float() + residual.float()).to(x.dtype))
        h = residual
    hf = h.float()
    w = weight.float() + 1.0 if gemma else weight.float()
    y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * w).to(x.dtype)
    packed, sfb = quantize_ref(y, gscale)
    return Nvfp4Tensor(packed, swizzle_sf(sfb), gscale, m, k), (y if want_normed else None)
