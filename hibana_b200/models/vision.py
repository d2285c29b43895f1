"""Vision encoder (ViT with 16 x 16 patches) feeding image tokens to the language model.

patchify (a GEMM over flattened patches) + learned position embedding -> `depth` pre-norm transformer blocks
(LayerNorm, non-causal multi-head attention, GELU MLP) -> pixel shuffle (2 x 2 neighbouring patches concatenated: 4x
fewer, 4x wider tokens) -> two-layer projector into the language model's hidden size. The GEMMs are the tcgen05 bf16
kernel and the attention is the tcgen05 prefill kernel run non-causally over a throw-away identity block table (head
dims that are not 64 or 128, e.g. ViT-H's 80, are zero-padded to 128: scores and outputs are unchanged).
Reference: hibana/model/nemotron/vision.py:1-164 (ViT-H/16 + pixel shuffle), hibana/engine/media.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..ops import attention, gemm


@dataclass(frozen=True)
class VisionConfig:
    image: int = 224
    patch: int = 16
    width: int = 1280
    depth: int = 32
    heads: int = 16
    mlp: int = 5120
    shuffle: int = 2          # pixel-shuffle factor per side
    out_hidden: int = 4096    # language-model hidden size
    eps: float = 1e-6

    @property
    def grid(self) -> int:
        return self.image // self.patch

    @property
    def tokens_per_image(self) -> int:
        return (self.grid // self.shuffle) ** 2


class VisionEncoder:
    def __init__(self, cfg: VisionConfig, device="cpu", seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator().manual_seed(seed)
        bf = lambda *s, std=0.02: (torch.randn(*s, generator=g) * std).to(torch.bfloat16).to(self.device)  # noqa: E731
        one = lambda n: torch.ones(n, dtype=torch.float32, device=self.device)  # noqa: E731
        zero = lambda n: torch.zeros(n, dtype=torch.float32, device=self.device)  # noqa: E731
        w, p = cfg.width, cfg.patch
        self.patch_w = bf(w, 3 * p * p)
        self.pos = bf(cfg.grid * cfg.grid, w)
        self.blocks = [{"ln1": (one(w), zero(w)), "qkv": bf(3 * w, w), "proj": bf(w, w), "ln2": (one(w), zero(w)),
                        "fc1": bf(cfg.mlp, w), "fc2": bf(w, cfg.mlp)} for _ in range(cfg.depth)]
        self.ln_out = (one(w), zero(w))
        wide = w * cfg.shuffle * cfg.shuffle
        self.proj1, self.proj2 = bf(cfg.out_hidden, wide), bf(cfg.out_hidden, cfg.out_hidden)
        self.tokens_per_image = cfg.tokens_per_image

    # ---- pieces
    def patchify(self, pixels: torch.Tensor) -> torch.Tensor:
        """[B, 3, S, S] -> [B * grid^2, 3 * p * p] rows in row-major patch order."""
        b, c, s, _ = pixels.shape
        p, gsz = self.cfg.patch, self.cfg.grid
        x = pixels.view(b, c, gsz, p, gsz, p).permute(0, 2, 4, 1, 3, 5).reshape(b * gsz * gsz, c * p * p)
        return x.to(torch.bfloat16).contiguous()

    def _attention(self, qkv: torch.Tensor, b: int, n: int) -> torch.Tensor:
        cfg = self.cfg
        hd = cfg.width // cfg.heads
        q, k, v = qkv.view(b * n, 3, cfg.heads, hd).unbind(1)
        scale = 1.0 / math.sqrt(hd)
        if not qkv.is_cuda:
            qq, kk, vv = (t.float().view(b, n, cfg.heads, hd).transpose(1, 2) for t in (q, k, v))
            out = F.scaled_dot_product_attention(qq, kk, vv, scale=scale)
            return out.transpose(1, 2).reshape(b * n, cfg.width).to(torch.bfloat16)
        d = 64 if hd <= 64 else 128
        pad = lambda t: F.pad(t, (0, d - hd)).contiguous() if d != hd else t.contiguous()  # noqa: E731
        q, k, v = pad(q), pad(k), pad(v)
        slots = torch.arange(b * n, dtype=torch.int32, device=qkv.device).view(b, n)
        ctx = torch.full((b,), n, dtype=torch.int32, device=qkv.device)
        indptr = (torch.arange(b + 1, device=qkv.device) * n).int()
        out = attention.paged_attention(q, k, v, slots, ctx, q_indptr=indptr, max_rows=n, scale=scale, causal=False)
        return out[..., :hd].reshape(b * n, cfg.width)

    def pixel_shuffle(self, x: torch.Tensor, b: int) -> torch.Tensor:
        """[B * g * g, W] -> [B * (g / s)^2, W * s * s]: the s x s neighbouring patches of a cell side by side."""
        gsz, s, w = self.cfg.grid, self.cfg.shuffle, self.cfg.width
        x = x.view(b, gsz // s, s, gsz // s, s, w).permute(0, 1, 3, 2, 4, 5)
        return x.reshape(b * (gsz // s) ** 2, s * s * w).contiguous()

    # ---- forward
    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, S, S] (float, normalised) -> image tokens [B * tokens_per_image, out_hidden] bf16."""
        cfg = self.cfg
        b = pixels.shape[0]
        n = cfg.grid * cfg.grid
        x = gemm.linear_bf16(self.patchify(pixels.to(self.device)), self.patch_w)
        x = (x.view(b, n, cfg.width) + self.pos).view(b * n, cfg.width)
        for blk in self.blocks:
            h = F.layer_norm(x.float(), (cfg.width,), *blk["ln1"], cfg.eps).to(torch.bfloat16)
            att = self._attention(gemm.linear_bf16(h, blk["qkv"]), b, n)
            x = gemm.linear_bf16(att, blk["proj"], epilogue=gemm.EPI_RESIDUAL, residual=x)
            h = F.layer_norm(x.float(), (cfg.width,), *blk["ln2"], cfg.eps).to(torch.bfloat16)
            m = F.gelu(gemm.linear_bf16(h, blk["fc1"]).float()).to(torch.bfloat16)
            x = gemm.linear_bf16(m, blk["fc2"], epilogue=gemm.EPI_RESIDUAL, residual=x)
        x = F.layer_norm(x.float(), (cfg.width,), *self.ln_out, cfg.eps).to(torch.bfloat16)
        x = self.pixel_shuffle(x, b)
        x = F.gelu(gemm.linear_bf16(x, self.proj1).float()).to(torch.bfloat16)
        return gemm.linear_bf16(x, self.proj2)
