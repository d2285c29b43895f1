"""Splits `<think>...</think>` reasoning from the visible answer, incrementally (reference:
hibana/api/parsers/reasoning.py)."""
from __future__ import annotations

OPEN, CLOSE = "<think>", "</think>"


class ReasoningParser:
    def __init__(self, starts_in_reasoning: bool = False):
        self.in_reasoning = starts_in_reasoning
        self.buf = ""

    def push(self, text: str) -> tuple[str, str]:
        """Returns (reasoning delta, content delta)."""
        self.buf += text
        reasoning, content = "", ""
        while self.buf:
            tag = CLOSE if self.in_reasoning else OPEN
            i = self.buf.find(tag)
            if i >= 0:
                piece, self.buf = self.buf[:i], self.buf[i + len(tag):]
                if self.in_reasoning:
                    reasoning += piece
                else:
                    content += piece
                self.in_reasoning = not self.in_reasoning
                continue
            # keep a possible partial tag at the end
            keep = 0
            for n in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-n:]):
                    keep = n
                    break
            piece, self.buf = self.buf[:len(self.buf) - keep], self.buf[len(self.buf) - keep:]
            if self.in_reasoning:
                reasoning += piece
            else:
                content += piece
            break
        return reasoning, content

    def flush(self) -> tuple[str, str]:
        piece, self.buf = self.buf, ""
        return (piece, "") if self.in_reasoning else ("", piece)
