"""Incremental detokeniser: emits only complete UTF-8 text as token ids arrive (reference: hibana/api/detok.py)."""
from __future__ import annotations


class IncrementalDetok:
    def __init__(self, tokenizer):
        self.tk = tokenizer
        self.ids: list[int] = []
        self.sent = 0          # bytes already emitted

    def push(self, new_ids) -> str:
        self.ids.extend(new_ids)
        data = self.tk.decode_bytes(self.ids)
        # hold back an incomplete trailing UTF-8 sequence
        end = len(data)
        for back in range(1, min(4, end) + 1):
            b = data[end - back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                end -= back
            break
        out = data[self.sent:end].decode("utf-8", errors="replace")
        self.sent = max(self.sent, end)
        return out

    def flush(self) -> str:
        data = self.tk.decode_bytes(self.ids)
        out = data[self.sent:].decode("utf-8", errors="replace")
        self.sent = len(data)
        return out
