"""3-bit weight copies ("w3") for bandwidth-bound decode.

Two logical formats:

* `Int3G64` — asymmetric 3-bit integer codes, groups of 64 along K, a bf16 scale and a bf16 zero point per
  (row, group): w ~= (code - zero) * scale. This is the format the benchmark configuration names and the one the
  dequant-fused GEMM (csrc/gemm.cu, kind w3) reads. Physical packing for the kernel is tile-major: for every
  (128-row block, 64-column group) one 4096-byte tile = 128 rows x 28 bytes of codes followed by 128 x (scale,
  zero) bf16 pairs, so a CTA fetches the tile with one bulk copy. Inside a row's 28 bytes, 32-bit word w holds codes
  10 w .. 10 w + 9: code 10 w + 2 i at bits [3 i, 3 i + 3) of the low half and code 10 w + 2 i + 1 at the same bits
  of the high half (bits 15 and 31 unused), which lets the kernel turn two codes into two bf16 values with one
  logic op (mask | 0x4300: the bf16 bit pattern of 128 + code) and two packed bf16 arithmetic ops.
  Storage: 3.5 bits of codes + 0.5 bits of scale / zero per weight.

* `CodebookW3` — the reference's logical content: 3-bit indices into an 8-entry codebook (per matrix), an e4m3 scale
  per 32 columns, an fp32 scale per row: w = codebook[code] * scale_e4m3[row, k // 32] * row_scale[row]; codes
  stored as three bit planes per 32-column word. Kept so that reference w3 checkpoints can be represented and
  dequantised; `to_int3g64` re-fits it onto the kernel's format (lossy only in the re-fit of non-uniform levels).
  The reference stores its planes in a mma-fragment-interleaved order specific to its sm_121 kernel
  (hibana/kernels/w3.py:200-230); that physical permutation is not reproduced here, the planes below are in plain
  row-major (row, 32-column word) order.
Reference: hibana/kernels/w3.py:239 (dequantize), hibana/weights/w3_checkpoint.py:104-160, docs/w3-calibration.md:3-12.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

GROUP = 64
WORDS = 7            # 32-bit words of codes per row and group
ROW_BYTES = 28
TILE_BYTES = 128 * ROW_BYTES + 128 * 4


@dataclass
class Int3G64:
    codes: torch.Tensor      # uint8 [N, K] values 0..7 (canonical, unpacked)
    scale: torch.Tensor      # bf16 [N, K / 64]
    zero: torch.Tensor       # bf16 [N, K / 64]

    @property
    def shape(self):
        return tuple(self.codes.shape)

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "Int3G64":
        n, k = w.shape
        assert k % GROUP == 0
        g = w.float().view(n, k // GROUP, GROUP)
        lo, hi = g.amin(-1), g.amax(-1)
        scale = ((hi - lo) / 7.0).clamp_min(1e-8).to(torch.bfloat16)
        zero = (-lo / scale.float()).to(torch.bfloat16)
        codes = torch.round(g / scale.float()[..., None] + zero.float()[..., None]).clamp(0, 7).to(torch.uint8)
        return cls(codes.view(n, k), scale, zero)

    def dequantize(self) -> torch.Tensor:
        """fp32 [N, K], with the kernel's arithmetic: bf16((code - zero) * scale) evaluated as
        fma(code, scale, bf16(-zero * scale)) in bf16."""
        n, k = self.codes.shape
        s = self.scale.float()[..., None]
        bias = (-(self.zero.float() * self.scale.float())).to(torch.bfloat16).float()[..., None]
        c = self.codes.view(n, k // GROUP, GROUP).float()
        return (c * s + bias).to(torch.bfloat16).float().view(n, k)

    def tiles(self) -> torch.Tensor:
        """Tile-major packing for the kernel: uint8 [N / 128, K / 64, 4096] (N padded to 128 with zero rows)."""
        n, k = self.codes.shape
        npad = (n + 127) // 128 * 128
        codes = torch.zeros(npad, k, dtype=torch.int32, device=self.codes.device)
        codes[:n] = self.codes.int()
        c = codes.view(npad, k // GROUP, GROUP)
        padded = torch.zeros(npad, k // GROUP, WORDS * 10, dtype=torch.int32, device=c.device)
        padded[..., :GROUP] = c
        p = padded.view(npad, k // GROUP, WORDS, 5, 2)            # [.., word, i, (low, high)]
        shifts = (3 * torch.arange(5, device=c.device)).view(1, 1, 1, 5)
        words = ((p[..., 0] << shifts) | (p[..., 1] << (shifts + 16))).sum(-1)      # int32 [npad, groups, 7]
        wbytes = words.to(torch.int64).view(npad, k // GROUP, WORDS, 1) >> (8 * torch.arange(4, device=c.device)) & 0xFF
        wbytes = wbytes.to(torch.uint8).view(npad, k // GROUP, ROW_BYTES)
        sz = torch.zeros(npad, k // GROUP, 2, dtype=torch.bfloat16, device=c.device)
        sz[:n, :, 0] = self.scale
        sz[:n, :, 1] = (-(self.zero.float() * self.scale.float())).to(torch.bfloat16)   # the kernel's bias term
        szb = sz.view(torch.uint8).view(npad, k // GROUP, 4)
        t_codes = wbytes.view(npad // 128, 128, k // GROUP, ROW_BYTES).permute(0, 2, 1, 3).reshape(npad // 128, k // GROUP, -1)
        t_sz = szb.view(npad // 128, 128, k // GROUP, 4).permute(0, 2, 1, 3).reshape(npad // 128, k // GROUP, -1)
        return torch.cat((t_codes, t_sz), dim=-1).contiguous()


@dataclass
class CodebookW3:
    planes: torch.Tensor     # int32 [N, K / 32, 3]: bit j of planes[r, w, p] = bit p of the code of column 32 w + j
    scales: torch.Tensor     # uint8 (e4m3 bits) [N, K / 32]
    row_scale: torch.Tensor  # fp32 [N]
    codebook: Sequence[float]

    @classmethod
    def pack(cls, codes: torch.Tensor, scales_e4m3: torch.Tensor, row_scale: torch.Tensor,
             codebook: Sequence[float]) -> "CodebookW3":
        n, k = codes.shape
        c = codes.int().view(n, k // 32, 32)
        bit = torch.arange(32, device=codes.device)
        planes = torch.stack([(((c >> p) & 1).to(torch.int64) << bit).sum(-1) for p in range(3)], dim=-1)
        planes = torch.where(planes >= 2 ** 31, planes - 2 ** 32, planes).to(torch.int32)
        return cls(planes, scales_e4m3.view(torch.uint8), row_scale.float(), tuple(codebook))

    def codes(self) -> torch.Tensor:
        bit = torch.arange(32, device=self.planes.device)
        pl = self.planes.to(torch.int64) & 0xFFFFFFFF
        c = sum((((pl[..., p, None] >> bit) & 1) << p) for p in range(3))
        return c.view(self.planes.shape[0], -1).to(torch.uint8)

    def dequantize(self) -> torch.Tensor:
        lv = torch.tensor(self.codebook, dtype=torch.float32, device=self.planes.device)
        sc = self.scales.view(torch.float8_e4m3fn).float() * self.row_scale[:, None]
        return lv[self.codes().long()] * sc.repeat_interleave(32, dim=1)

    def to_int3g64(self) -> Int3G64:
        return Int3G64.quantize(self.dequantize())
