"""Image parts of chat requests (OpenAI `image_url` / `input_image`, Anthropic `image` blocks) for targets that
carry a vision encoder.

Images must come inline (a `data:` URL or a base64 source): the server fetches nothing. `prepare` walks the
messages, replaces every image part by the text marker the chat template understands, and returns the images in
order; text that happens to contain the marker is escaped so it cannot claim an image. After the template is
rendered and tokenised, `expand` replaces each marker token run by the image's placeholder ids (negative ids derived
from the image bytes, engine/media.py), which is what lets the radix prefix cache match a conversation that carries
the same image again. The engine encodes an image only when its placeholder span is actually prefilled.
Reference: hibana/api/media.py:36-172.
"""
from __future__ import annotations

import base64
import binascii
from dataclasses import dataclass, field
from typing import Optional

from ..engine.media import Image, placeholder_ids
from .validation import BadRequest

MARKER = "<image>"
_ESCAPE = "image>"            # private-use stand-in for "<" while user text travels through the template
MAX_IMAGE_BYTES = 32 << 20
MAX_IMAGES = 100
IMAGE_KINDS = ("image_url", "input_image", "image")


@dataclass
class MediaPlan:
    """What the engine needs to splice image embeddings into a prompt: the images and, once `expand` ran, the
    (start position, token count) of each image's placeholder span in the prompt."""
    images: list = field(default_factory=list)
    spans: list = field(default_factory=list)


def _decode_b64(data) -> bytes:
    if not isinstance(data, str) or not data:
        raise BadRequest("image data must be a base64 string")
    try:
        raw = base64.b64decode(data, validate=False)
    except (binascii.Error, ValueError):
        raise BadRequest("image data is not valid base64") from None
    if not raw or len(raw) > MAX_IMAGE_BYTES:
        raise BadRequest("image is empty or larger than 32 MiB")
    return raw


def image_bytes(part: dict) -> bytes:
    """Encoded bytes of one image part."""
    if part.get("type") == "image":                         # Anthropic block
        src = part.get("source")
        if not isinstance(src, dict):
            raise BadRequest("an image block needs a source")
        if src.get("type") == "base64":
            return _decode_b64(src.get("data"))
        url = src.get("url")
    else:                                                   # OpenAI chat part or Responses-style input_image
        url = part.get("image_url")
        url = url.get("url") if isinstance(url, dict) else url
    if not isinstance(url, str) or not url.startswith("data:"):
        raise BadRequest("images must be sent inline (data: URL or base64); this server does not fetch URLs")
    head, _, data = url.partition(",")
    if not head.endswith(";base64"):
        raise BadRequest("a data: URL image must be base64 encoded")
    return _decode_b64(data)


def prepare(messages: list) -> tuple[list, MediaPlan]:
    """Returns (messages with image parts turned into marker text, plan holding the images in order)."""
    plan = MediaPlan()
    out = []
    for m in messages:
        content = m.get("content") if isinstance(m, dict) else None
        if isinstance(content, str):
            out.append(dict(m, content=content.replace(MARKER, _ESCAPE)))
            continue
        if not isinstance(content, list):
            out.append(m)
            continue
        pieces = []
        for part in content:
            if isinstance(part, dict) and part.get("type") in IMAGE_KINDS:
                if len(plan.images) >= MAX_IMAGES:
                    raise BadRequest(f"at most {MAX_IMAGES} images per request")
                plan.images.append(Image(image_bytes(part), None))
                pieces.append(MARKER)
            elif isinstance(part, dict) and part.get("type") in ("text", "input_text"):
                pieces.append(str(part.get("text", "")).replace(MARKER, _ESCAPE))
        out.append(dict(m, content="".join(pieces)))
    return out, plan


def unescape(text: str) -> str:
    return text.replace(_ESCAPE, MARKER)


def expand(text: str, tokenizer, plan: MediaPlan, tokens_per_image: int) -> list:
    """Tokenises the rendered prompt piecewise around the markers and puts each image's placeholder ids where its
    marker stood; fills `plan.spans`."""
    chunks = text.split(MARKER)
    if len(chunks) - 1 != len(plan.images):
        raise BadRequest("the chat template did not place every image exactly once")
    ids: list = []
    plan.spans = []
    for i, chunk in enumerate(chunks):
        if chunk:
            ids.extend(tokenizer.encode(unescape(chunk)))
        if i < len(plan.images):
            plan.spans.append((len(ids), tokens_per_image))
            ids.extend(placeholder_ids(plan.images[i], tokens_per_image))
    return ids


def strip_images(messages: list, note: str = "[image omitted: this model takes no images]") -> list:
    """For targets without a vision encoder: image parts become a short note instead of failing the request."""
    out = []
    for m in messages:
        content = m.get("content") if isinstance(m, dict) else None
        if isinstance(content, list):
            text = "".join(note if isinstance(p, dict) and p.get("type") in IMAGE_KINDS else str(p.get("text", ""))
                           for p in content if isinstance(p, dict))
            out.append(dict(m, content=text))
        else:
            out.append(m)
    return out


def has_images(messages: list) -> bool:
    return any(isinstance(m, dict) and isinstance(m.get("content"), list)
               and any(isinstance(p, dict) and p.get("type") in IMAGE_KINDS for p in m["content"]) for m in messages)
