"""Tokenizers: a Hugging Face `tokenizer.json` when a checkpoint directory has one, else a byte-level fallback.

The fallback maps UTF-8 bytes to ids 3..258 (0 = pad, 1 = bos, 2 = eos) so a random-init model can be served and
tested offline. Reference: hibana/tokenizer.py (snapshot tokenizer wrapper).
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence


class ByteTokenizer:
    pad_id, bos_id, eos_id = 0, 1, 2
    OFFSET = 3

    def __init__(self, vocab: int = 259):
        self.vocab_size = max(vocab, 259)

    def encode(self, text: str, add_bos: bool = False) -> list[int]:
        ids = [b + self.OFFSET for b in text.encode("utf-8")]
        return ([self.bos_id] + ids) if add_bos else ids

    def decode(self, ids: Sequence[int]) -> str:
        data = bytes((i - self.OFFSET) & 0xFF for i in ids if self.OFFSET <= i < self.OFFSET + 256)
        return data.decode("utf-8", errors="replace")

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return bytes((i - self.OFFSET) & 0xFF for i in ids if self.OFFSET <= i < self.OFFSET + 256)


class HfTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        self.eos_id = self.tk.token_to_id("<|im_end|>") or self.tk.token_to_id("</s>") or 2
        self.bos_id = self.tk.token_to_id("<s>")
        self.pad_id = 0

    def encode(self, text: str, add_bos: bool = False) -> list[int]:
        ids = self.tk.encode(text, add_special_tokens=False).ids
        return ([self.bos_id] + ids) if add_bos and self.bos_id is not None else ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=True)

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return self.decode(ids).encode("utf-8")


def load_tokenizer(checkpoint: Optional[str], vocab: int):
    if checkpoint:
        f = Path(checkpoint) / "tokenizer.json"
        if f.exists():
            return HfTokenizer(str(f))
    return ByteTokenizer(vocab)
