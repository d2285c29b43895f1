"""Reader of the reference's calibrated 3-bit checkpoint directories.

A directory holds `manifest.json` ({"format": 1, "target_revision": ..., "weights": {name: {"file", "sha256",
"out_features", "in_features", "codebook"}}}) and one safetensors file per matrix with three tensors:

    planes     uint32 [N / 32, K / 128, bits, 32, 4]   bit planes of the codes, in the order the reference's
                                                        mma.sync fragments consume them
    scales     uint8  [N / 32, K / 128, 4, 32]          e4m3 scale of every (row, 32-column group)
    row_scale  fp32   [N]

The weight is codebook[code] * scale * row_scale. Physical order (read from the reference's packer, restated):
row n = 32 nb + 8 nt + g, column k = 128 kc + 16 s + 4 t + j. Bit b of that weight's code sits in
planes[nb, kc, b, lane = 4 g + t, nt] at bit position (4 j + b + rot(s)) mod 32 with rot(s) = 16 (s // 4) + s % 4.
The scale of row n = 32 nb + 8 nt + 2 t + i, group 4 kc + grp is scales[nb, kc, t, 8 nt + 2 grp + i].

`ReferenceW3Checkpoint.load(name)` checks the file against the manifest's SHA-256, undoes that order and returns a
`CodebookW3` (codes, e4m3 scales, row scales in plain row-major order): the same numbers, nothing re-fitted.
`CodebookLinear` serves them without requantising: the tensor-core operand is codebook[code] * scale, which is exact
in bf16 (two 4-bit significands), and the fp32 row scale multiplies the fp32-accumulated output. `write_directory`
writes the same format (fixtures, and copies calibrated by this build).
Reference: hibana/weights/w3_checkpoint.py:57-140, hibana/kernels/w3.py:1-36,147-237.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Optional, Sequence

import torch

from .w3 import CodebookW3

FORMAT_VERSION = 1
MANIFEST = "manifest.json"


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(8 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _rot(device) -> torch.Tensor:
    s = torch.arange(8, device=device)
    return 16 * (s // 4) + (s % 4)


def _bit_positions(b: int, device) -> torch.Tensor:
    """[s, j] -> position of bit b of the code of column 16 s + 4 t + j inside its plane word."""
    j = torch.arange(4, device=device)
    return (4 * j[None, :] + b + _rot(device)[:, None]) % 32


def decode_planes(planes: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """planes [N / 32, K / 128, bits, 32, 4] -> codes uint8 [N, K]."""
    nb, kc, bits = n // 32, k // 128, planes.shape[2]
    w = planes.to(torch.int64) & 0xFFFFFFFF
    w = w.view(nb, kc, bits, 8, 4, 4)                       # [nb, kc, b, g, t, nt]
    codes = torch.zeros(nb, 4, 8, kc, 8, 4, 4, dtype=torch.int64, device=planes.device)   # [nb, nt, g, kc, s, t, j]
    for b in range(bits):
        pos = _bit_positions(b, planes.device)              # [s, j]
        word = w[:, :, b].permute(0, 4, 2, 1, 3)            # [nb, nt, g, kc, t]
        bit = (word[:, :, :, :, None, :, None] >> pos[None, None, None, None, :, None, :]) & 1
        codes |= bit << b
    return codes.reshape(n, k).to(torch.uint8)


def encode_planes(codes: torch.Tensor, bits: int = 3) -> torch.Tensor:
    """codes [N, K] -> planes uint32 [N / 32, K / 128, bits, 32, 4] (the inverse of `decode_planes`)."""
    n, k = codes.shape
    q = codes.to(torch.int64).view(n // 32, 4, 8, k // 128, 8, 4, 4)      # [nb, nt, g, kc, s, t, j]
    out = torch.zeros(n // 32, k // 128, bits, 32, 4, dtype=torch.int64, device=codes.device)
    for b in range(bits):
        pos = _bit_positions(b, codes.device)
        word = (((q >> b) & 1) << pos[None, None, None, None, :, None, :]).sum(dim=(4, 6))    # [nb, nt, g, kc, t]
        out[:, :, b] = word.permute(0, 3, 2, 4, 1).reshape(n // 32, k // 128, 32, 4)           # lane = 4 g + t, nt
    return out.to(torch.uint32)


def decode_scales(scales: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """scales uint8 [N / 32, K / 128, 4, 32] -> e4m3 bits [N, K / 32] in row-major order."""
    s = scales.view(n // 32, k // 128, 4, 4, 4, 2)          # [nb, kc, t, nt, grp, i]
    return s.permute(0, 3, 2, 5, 1, 4).reshape(n, k // 32).contiguous()


def encode_scales(sc: torch.Tensor) -> torch.Tensor:
    n, groups = sc.shape
    s = sc.view(n // 32, 4, 4, 2, groups // 4, 4)           # [nb, nt, t, i, kc, grp]
    return s.permute(0, 4, 2, 1, 5, 3).reshape(n // 32, groups // 4, 4, 32).contiguous()


class ReferenceW3Checkpoint:
    def __init__(self, directory: str | Path, revision: Optional[str] = None):
        self.directory = Path(directory)
        path = self.directory / MANIFEST
        if not path.is_file():
            raise FileNotFoundError(f"{self.directory} has no {MANIFEST}: not a calibrated 3-bit checkpoint")
        self.manifest = json.loads(path.read_text())
        if self.manifest.get("format") != FORMAT_VERSION:
            raise ValueError(f"3-bit checkpoint format {self.manifest.get('format')!r}, this reader knows {FORMAT_VERSION}")
        if revision is not None and self.manifest.get("target_revision") != revision:
            raise ValueError("the 3-bit checkpoint was calibrated for another revision of the target")
        self.weights: dict = self.manifest["weights"]
        self.identity = sha256_file(path)

    def names(self) -> list[str]:
        return sorted(self.weights)

    def expert_layers(self) -> set[int]:
        return {int(n.split(".")[1]) for n in self.weights if n.startswith("layers.") and ".experts." in n}

    def _entry(self, name: str) -> tuple[dict, Path]:
        entry = self.weights[name]
        fname = entry["file"]
        if Path(fname).name != fname:
            raise ValueError("3-bit checkpoint files must sit directly inside the directory")
        return entry, self.directory / fname

    def verify(self, name: Optional[str] = None) -> None:
        """Raises when a file's SHA-256 differs from the manifest (all files when `name` is None)."""
        for nm in ([name] if name else self.names()):
            entry, path = self._entry(nm)
            if sha256_file(path) != entry["sha256"]:
                raise ValueError(f"checksum mismatch for {nm} ({path.name})")

    def load(self, name: str, device="cpu", verify: bool = True, rows: Optional[slice] = None) -> CodebookW3:
        """The matrix `name` (its row range `rows`, a multiple of 32, under tensor parallelism)."""
        from safetensors import safe_open
        entry, path = self._entry(name)
        if verify and sha256_file(path) != entry["sha256"]:
            raise ValueError(f"checksum mismatch for {name} ({path.name})")
        n, k = int(entry["out_features"]), int(entry["in_features"])
        with safe_open(str(path), framework="pt") as f:
            if set(f.keys()) != {"planes", "scales", "row_scale"}:
                raise ValueError(f"{path.name}: expected planes / scales / row_scale")
            planes, scales, row_scale = f.get_tensor("planes"), f.get_tensor("scales"), f.get_tensor("row_scale")
        bits = planes.shape[2]
        want = {"planes": (n // 32, k // 128, bits, 32, 4), "scales": (n // 32, k // 128, 4, 32), "row_scale": (n,)}
        if (tuple(planes.shape), tuple(scales.shape), tuple(row_scale.shape)) != tuple(want.values()) or bits not in (2, 3):
            raise ValueError(f"{path.name}: tensor shapes do not match the manifest's {n} x {k}")
        levels = _codebook(entry.get("codebook"))
        if len(levels) != (1 << bits):
            raise ValueError(f"{name}: {len(levels)} codebook levels for {bits}-bit codes")
        if rows is not None:
            lo, hi = rows.start or 0, rows.stop if rows.stop is not None else n
            if lo % 32 or hi % 32:
                raise ValueError("row ranges must fall on 32-row blocks")
            planes, scales, row_scale = planes[lo // 32:hi // 32], scales[lo // 32:hi // 32], row_scale[lo:hi]
            n = hi - lo
        codes = decode_planes(planes, n, k)
        sc = decode_scales(scales, n, k)
        return CodebookW3.pack(codes.to(device), sc.to(device).view(torch.float8_e4m3fn), row_scale.to(device), levels)


CODEBOOKS = {"uniform": (-3.5, -2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 3.5)}


def _codebook(cb) -> tuple:
    if isinstance(cb, str):
        if cb not in CODEBOOKS:
            raise ValueError(f"the manifest names codebook {cb!r} without its levels")
        return CODEBOOKS[cb]
    levels = tuple(float(v) for v in (cb or CODEBOOKS["uniform"]))
    if len(levels) not in (4, 8) or list(levels) != sorted(levels):
        raise ValueError("a codebook is four or eight ascending levels")
    return levels


def write_directory(directory: str | Path, weights: dict, revision: str = "local") -> Path:
    """weights: {name: CodebookW3}. Writes the reference's directory format (N % 128 == 0, K % 128 == 0)."""
    from safetensors.torch import save_file
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    manifest = {"format": FORMAT_VERSION, "target_revision": revision, "weights": {}}
    for i, (name, w) in enumerate(sorted(weights.items())):
        codes = w.codes()
        n, k = codes.shape
        if n % 128 or k % 128:
            raise ValueError(f"{name}: {n} x {k} is not a multiple of 128 in both dimensions")
        bits = 2 if len(w.codebook) == 4 else 3
        fname = f"w3-{i:05d}.safetensors"
        save_file({"planes": encode_planes(codes.cpu(), bits).contiguous(),
                   "scales": encode_scales(w.scales.cpu().view(torch.uint8)),
                   "row_scale": w.row_scale.cpu().float().contiguous()}, str(d / fname))
        manifest["weights"][name] = {"file": fname, "sha256": sha256_file(d / fname), "out_features": n,
                                     "in_features": k, "codebook": list(w.codebook)}
    (d / MANIFEST).write_text(json.dumps(manifest, indent=1))
    return d


class CodebookLinear:
    """y = x @ W.T for a `CodebookW3` matrix without touching its codes or scales: the GEMM operand is
    codebook[code] * group scale (exact in bf16) and the fp32 row scale multiplies the fp32-accumulated result."""

    def __init__(self, w: CodebookW3, device=None, name: str = ""):
        dev = torch.device(device) if device is not None else w.planes.device
        lv = torch.tensor(w.codebook, dtype=torch.float32, device=w.planes.device)
        sc = w.scales.view(torch.float8_e4m3fn).float()
        unit = lv[w.codes().long()] * sc.repeat_interleave(32, dim=1)
        self.weight = unit.to(torch.bfloat16).to(dev).contiguous()
        assert torch.equal(self.weight.float().cpu(), unit.cpu()), "level x e4m3 scale must be exact in bf16"
        self.row_scale = w.row_scale.float().to(dev)
        self.out_features, self.in_features = self.weight.shape
        self.name, self.fmt = name, "w3-codebook"

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import gemm
        y = gemm.linear_bf16(x, self.weight, epilogue=gemm.EPI_STORE_F32)
        return (y * self.row_scale).to(torch.bfloat16)

    def nbytes(self) -> int:
        return self.weight.numel() * 2 + self.row_scale.numel() * 4


def current_checkpoint(root: str | Path, target: str) -> Optional[Path]:
    """`<root>/<target>-current` when it holds a complete checkpoint (the link the reference's launcher serves)."""
    link = Path(root) / f"{target}-current"
    return link.resolve() if (link / MANIFEST).is_file() else None
