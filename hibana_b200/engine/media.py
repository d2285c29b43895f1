"""Images in prompts: every image becomes `tokens_per_image` placeholder token ids that (a) are negative, so they can
never collide with vocabulary ids, and (b) derive from a hash of the image bytes, so the radix prefix cache matches
two requests carrying the same image and never confuses different ones. At prefill the embedding rows of the
placeholders are replaced by the vision encoder's output. Reference: hibana/engine/media.py:1-178 (placeholder ids from
shake_256), hibana/api/media.py:87-172 (prepare / expand).
"""
from __future__ import annotations

import base64
import hashlib
from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class Image:
    data: bytes                       # encoded or raw bytes as received (hashed for the placeholder ids)
    pixels: Optional[torch.Tensor]    # [3, S, S] float, normalised; None until decoded

    @classmethod
    def from_data_url(cls, url: str) -> "Image":
        if not url.startswith("data:") or ";base64," not in url:
            raise ValueError("images must be data: URLs with base64 payload")
        return cls(base64.b64decode(url.split(";base64,", 1)[1]), None)


def placeholder_ids(image: Image, count: int) -> list[int]:
    """`count` distinct negative ids derived from the image content."""
    raw = hashlib.shake_256(image.data).digest(8 * count)
    ids = []
    for i in range(count):
        v = int.from_bytes(raw[8 * i:8 * i + 8], "little") & ((1 << 62) - 1)
        ids.append(-(v + 1))
    return ids


def expand(token_ids: Sequence[int], image_token: int, images: Sequence[Image], tokens_per_image: int) -> list[int]:
    """Replaces every occurrence of the tokenizer's image token by the image's placeholder ids (in order)."""
    out, it = [], iter(images)
    for t in token_ids:
        if t == image_token:
            try:
                img = next(it)
            except StopIteration:
                raise ValueError("more image tokens than images") from None
            out.extend(placeholder_ids(img, tokens_per_image))
        else:
            out.append(t)
    if next(it, None) is not None:
        raise ValueError("more images than image tokens")
    return out


def splice_embeddings(ids: torch.Tensor, embeds: torch.Tensor, image_embeds: torch.Tensor) -> torch.Tensor:
    """Rows of `embeds` at negative ids are replaced, in order, by the rows of `image_embeds`."""
    mask = ids < 0
    if int(mask.sum()) != image_embeds.shape[0]:
        raise ValueError("placeholder count does not match the encoder output")
    out = embeds.clone()
    out[mask] = image_embeds.to(embeds.dtype)
    return out


def decode_pixels(image: Image, size: int) -> torch.Tensor:
    """Encoded bytes (PNG / JPEG / anything Pillow reads) -> [3, size, size] float pixels, resized and normalised to
    mean 0.5 / std 0.5. Cached on the image."""
    if image.pixels is not None and image.pixels.shape[-1] == size:
        return image.pixels
    import io

    import numpy as np
    from PIL import Image as PilImage
    try:
        pic = PilImage.open(io.BytesIO(image.data)).convert("RGB").resize((size, size), PilImage.BICUBIC)
    except Exception as e:  # noqa: BLE001
        raise ValueError(f"image does not decode: {e}") from None
    arr = torch.from_numpy(np.asarray(pic, dtype=np.float32) / 255.0).permute(2, 0, 1)
    image.pixels = (arr - 0.5) / 0.5
    return image.pixels


class VisionCache:
    """Encoder outputs by image content (a conversation sends the same image again with every turn, and a long
    prefill touches an image's span in several chunks); least recently used entries go first."""

    def __init__(self, encoder, capacity: int = 64):
        self.encoder, self.capacity = encoder, capacity
        self.rows: dict = {}

    def embeddings(self, image: Image) -> torch.Tensor:
        key = hashlib.sha256(image.data).digest()
        hit = self.rows.pop(key, None)
        if hit is None:
            px = decode_pixels(image, self.encoder.cfg.image)
            hit = self.encoder.encode(px[None])
            while len(self.rows) >= self.capacity:
                self.rows.pop(next(iter(self.rows)))
        self.rows[key] = hit
        return hit


def chunk_embeddings(plan, start: int, count: int, cache: VisionCache) -> Optional[torch.Tensor]:
    """Image-embedding rows for the placeholder positions inside prompt positions [start, start + count), in
    order (None when the chunk holds none). `plan` is an api/media.MediaPlan (images + spans)."""
    rows = []
    for img, (pos, n) in zip(plan.images, plan.spans):
        lo, hi = max(pos, start), min(pos + n, start + count)
        if lo < hi:
            rows.append(cache.embeddings(img)[lo - pos:hi - pos])
    return torch.cat(rows, 0) if rows else None
