"""GGUF container reader and GGML block codecs (the formats Bolt-class checkpoints ship in).

`GgufFile` parses a GGUF v2 / v3 file (little endian): header, typed key-value metadata, tensor directory, aligned
data section, and hands out tensors as zero-copy numpy views of a memory map. `dequantize` turns the block formats
this build decodes into fp32:

* F32, F16, BF16 — plain;
* Q8_0 — blocks of 32 weights: one fp16 scale d and 32 int8 codes, w = d * q (34 bytes per block);
* IQ2_XXS / IQ2_XS — 256-weight super-blocks: an fp16 scale and 2.06 / 2.31 bits per weight as indices into an E8
  lattice codebook (256 / 512 entries of 8 magnitudes) plus 7 sign bits per 8 weights (the eighth sign makes the
  parity even) and a 4-bit sub-scale. The lattice tables are part of the format, not of this file: pass them as
  `grids={"iq2_xxs": uint8 [256, 8], "iq2_xs": uint8 [512, 8]}` (e.g. loaded from a .npy next to the checkpoint);
  without them these two types raise a clear error instead of decoding wrongly.

Decoded matrices feed the normal loaders (bf16 / NVFP4 / int3-g64 re-quantisation); a decode-fused IQ2 grouped GEMM
like the reference's is not built. `write_gguf` writes small files (tests, fixtures).
Reference: hibana/weights/ggml.py (dequantisers), hibana/kernels/ggml.py:1-84, hibana/kernels/csrc/ggml_codec.cuh.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Optional

import numpy as np

GGUF_MAGIC = b"GGUF"
T_F32, T_F16, T_Q8_0, T_IQ2_XXS, T_IQ2_XS, T_BF16 = 0, 1, 8, 16, 17, 30
# type -> (weights per block, bytes per block)
BLOCK = {T_F32: (1, 4), T_F16: (1, 2), T_BF16: (1, 2), T_Q8_0: (32, 34), T_IQ2_XXS: (256, 66), T_IQ2_XS: (256, 74)}
NAMES = {T_F32: "f32", T_F16: "f16", T_BF16: "bf16", T_Q8_0: "q8_0", T_IQ2_XXS: "iq2_xxs", T_IQ2_XS: "iq2_xs"}

_KV_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
KV_STRING, KV_ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    shape: tuple          # logical shape, outermost first (GGUF stores innermost first)
    dtype: int
    offset: int           # from the start of the data section

    @property
    def nbytes(self) -> int:
        per, size = BLOCK[self.dtype]
        n = int(np.prod(self.shape))
        assert n % per == 0
        return n // per * size


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, kind: int):
        if kind == KV_STRING:
            return self.string()
        if kind == KV_ARRAY:
            sub, n = self.take("<I"), self.take("<Q")
            return [self.value(sub) for _ in range(n)]
        if kind not in _KV_FMT:
            raise ValueError(f"unknown GGUF value type {kind}")
        return self.take(_KV_FMT[kind])


class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(self._mm)
        if bytes(self._mm[:4]) != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        r.pos = 4
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.meta: dict = {}
        for _ in range(n_kv):
            key = r.string()
            self.meta[key] = r.value(r.take("<I"))
        self.tensors: dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<Q") for _ in range(nd)]
            dtype, off = r.take("<I"), r.take("<Q")
            if dtype not in BLOCK:
                raise ValueError(f"{path}: tensor {name} has GGML type {dtype}, which this build does not decode")
            self.tensors[name] = TensorInfo(name, tuple(reversed(dims)), dtype, off)
        align = int(self.meta.get("general.alignment", 32))
        self.data_start = (r.pos + align - 1) // align * align

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        start = self.data_start + t.offset
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=start)

    def load(self, name: str, grids: Optional[dict] = None) -> np.ndarray:
        t = self.tensors[name]
        return dequantize(self.raw(name), t.dtype, t.shape, grids)

    def close(self) -> None:
        self._mm.close()
        self._fh.close()


def _ksigns() -> np.ndarray:
    """7 stored sign bits -> 8 signs: the eighth makes the number of negative signs even."""
    i = np.arange(128, dtype=np.uint16)
    par = np.zeros(128, dtype=np.uint16)
    for b in range(7):
        par ^= (i >> b) & 1
    return (i | (par << 7)).astype(np.uint8)


def dequantize(raw: np.ndarray, dtype: int, shape, grids: Optional[dict] = None) -> np.ndarray:
    """Raw block bytes -> fp32 array of `shape`."""
    n = int(np.prod(shape))
    if dtype == T_F32:
        return raw.view(np.float32).reshape(shape).copy()
    if dtype == T_F16:
        return raw.view(np.float16).astype(np.float32).reshape(shape)
    if dtype == T_BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
    if dtype == T_Q8_0:
        blk = raw.reshape(n // 32, 34)
        d = blk[:, :2].copy().view(np.float16).astype(np.float32)               # [blocks, 1]
        q = blk[:, 2:].view(np.int8).astype(np.float32)
        return (q * d).reshape(shape)
    if dtype in (T_IQ2_XXS, T_IQ2_XS):
        key = NAMES[dtype]
        if not grids or key not in grids:
            raise ValueError(f"decoding {key} needs the format's lattice table: pass grids={{'{key}': uint8 [N, 8]}}")
        grid = np.asarray(grids[key], dtype=np.float32)
        signs_tab = _ksigns()
        bits = np.arange(8, dtype=np.uint8)
        if dtype == T_IQ2_XXS:
            blk = raw.reshape(n // 256, 66)
            d = blk[:, :2].copy().view(np.float16).astype(np.float32)[:, 0]
            qs = blk[:, 2:].copy().view(np.uint32).reshape(-1, 8, 2)              # per 32 weights: indices, signs+scale
            idx = qs[..., 0:1].view(np.uint8).reshape(-1, 8, 4)                   # four grid indices
            aux = qs[..., 1]
            sc = (aux >> 28).astype(np.float32)
            sidx = np.stack([(aux >> (7 * j)) & 127 for j in range(4)], -1)      # [blocks, 8, 4]
            sg = signs_tab[sidx]
            neg = ((sg[..., None] >> bits) & 1).astype(np.float32)                # [blocks, 8, 4, 8]
            w = grid[idx] * (1.0 - 2.0 * neg)
            db = d[:, None] * (0.5 + sc) * 0.25
            return (w * db[:, :, None, None]).reshape(shape).astype(np.float32)
        blk = raw.reshape(n // 256, 74)
        d = blk[:, :2].copy().view(np.float16).astype(np.float32)[:, 0]
        qs = blk[:, 2:66].copy().view(np.uint16).reshape(-1, 8, 4)                # 9-bit index + 7 sign bits
        scales = blk[:, 66:74]                                                    # two 4-bit sub-scales per byte
        idx, sidx = qs & 511, qs >> 9
        neg = ((signs_tab[sidx][..., None] >> bits) & 1).astype(np.float32)
        w = grid[idx] * (1.0 - 2.0 * neg)                                         # [blocks, 8, 4, 8]
        sc = np.stack([scales & 15, scales >> 4], -1).astype(np.float32)          # [blocks, 8, 2]: per 16 weights
        db = d[:, None, None] * (0.5 + sc) * 0.25
        return (w * np.repeat(db, 2, axis=2)[..., None]).reshape(shape).astype(np.float32)
    raise ValueError(f"GGML type {dtype} is not decoded by this build")


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """fp32 [..., K] (K % 32 == 0) -> Q8_0 block bytes (round to nearest, scale = amax / 127)."""
    g = w.astype(np.float32).reshape(-1, 32)
    d = np.abs(g).max(1) / 127.0
    q = np.where(d[:, None] > 0, np.round(g / np.where(d > 0, d, 1)[:, None]), 0).astype(np.int8)
    out = np.empty((g.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def write_gguf(path: str, tensors: dict, meta: Optional[dict] = None, align: int = 32) -> None:
    """tensors: name -> (raw uint8 bytes, GGML type, logical shape). meta: str / int / float values."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    meta = dict(meta or {})
    meta.setdefault("general.alignment", align)
    head = GGUF_MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += s(k)
        if isinstance(v, str):
            head += struct.pack("<I", KV_STRING) + s(v)
        elif isinstance(v, float):
            head += struct.pack("<If", 6, v)
        else:
            head += struct.pack("<II", 4, int(v))
    blobs, off = [], 0
    for name, (raw, dtype, shape) in tensors.items():
        head += s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        head += struct.pack("<IQ", dtype, off)
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        blobs.append((off, raw))
        off = (off + raw.size + align - 1) // align * align
    start = (len(head) + align - 1) // align * align
    with open(path, "wb") as fh:
        fh.write(head + b"\0" * (start - len(head)))
        for o, raw in blobs:
            fh.seek(start + o)
            fh.write(raw.tobytes())
        fh.truncate(start + off)
