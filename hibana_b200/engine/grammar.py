"""Grammar-constrained output: a request's grammar as token bitmasks for the sampling kernels.

`Grammars` compiles a constraint once per (kind, source) with xgrammar (JSON schema, any JSON object, EBNF, regex or
forced tool calls); every request owns a `GrammarState` built from it. The state advances on each emitted token
(`push`) and supplies the allowed-token bitmask (int32 [ceil(vocab / 32)], bit i set = token i allowed) that the
argmax / sampling kernels (csrc/sample.cu) take next to the logits, so masking costs no extra pass over the
logits. For a speculative round, `verify_masks` walks the drafted tokens through the grammar and returns one mask
per verified row (the state after the drafted prefix before it), rolling the matcher back afterwards. Reasoning is
free: with `think_end` set the grammar applies from the first token after that id. Once the grammar is complete only
the stop tokens remain allowed. A constraint travels to other ranks as its source (`Constraint.source`), since a
compiled grammar does not pickle. Reference: hibana/engine/grammar.py:1-231.
"""
from __future__ import annotations

import json
import threading
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

try:
    import xgrammar as xgr
except ImportError:           # the serving paths report a clear error when a constraint is requested
    xgr = None

TOOL_CALL_EBNF = r'''
root ::= ws "<tool_call>" ws call ws "</tool_call>"
call ::= "{" ws "\"name\"" ws ":" ws string ws "," ws "\"arguments\"" ws ":" ws object ws "}"
object ::= "{" ws (pair (ws "," ws pair)*)? ws "}"
pair ::= string ws ":" ws value
array ::= "[" ws (value (ws "," ws value)*)? ws "]"
value ::= object | array | string | number | "true" | "false" | "null"
string ::= "\"" ([^"\\] | "\\" ["\\/bfnrt] | "\\u" [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F] [0-9a-fA-F])* "\""
number ::= "-"? ("0" | [1-9] [0-9]*) ("." [0-9]+)? ([eE] [-+]? [0-9]+)?
ws ::= [ \t\n]*
'''


@dataclass(frozen=True)
class Constraint:
    compiled: object              # xgrammar.CompiledGrammar (shareable between requests)
    kind: str                     # json_schema | json_object | ebnf | regex | tool_call
    source: str                   # what it was compiled from (sent to other ranks instead of `compiled`)
    think_end: Optional[int] = None   # token id that ends a reasoning block; None = the grammar applies at once


class Grammars:
    """Compiler + cache for one tokenizer. `vocab[i]` is the text (or bytes) of token i."""

    def __init__(self, vocab: Sequence, vocab_size: Optional[int] = None, stop_ids: Sequence[int] = ()):
        if xgr is None:
            raise RuntimeError("grammar-constrained output needs the xgrammar package")
        self.vocab_size = vocab_size or len(vocab)
        self.info = xgr.TokenizerInfo(list(vocab), vocab_size=self.vocab_size,
                                      stop_token_ids=list(stop_ids) if stop_ids else None)
        self.compiler = xgr.GrammarCompiler(self.info, max_threads=4)
        self.words = (self.vocab_size + 31) // 32
        self._cache: dict = {}
        self._lock = threading.Lock()

    def _get(self, kind: str, source: str, think_end: Optional[int]) -> Constraint:
        with self._lock:
            hit = self._cache.get((kind, source))
            if hit is None:
                if kind == "json_schema":
                    # compact JSON: with free whitespace a weak model can pad to its length limit without leaving the grammar
                    hit = self.compiler.compile_json_schema(source, any_whitespace=False)
                elif kind == "json_object":
                    hit = self.compiler.compile_builtin_json_grammar()
                elif kind == "regex":
                    hit = self.compiler.compile_regex(source)
                else:
                    hit = self.compiler.compile_grammar(source)
                self._cache[(kind, source)] = hit
        return Constraint(hit, kind, source, think_end)

    def json_schema(self, schema, think_end: Optional[int] = None) -> Constraint:
        return self._get("json_schema", schema if isinstance(schema, str) else json.dumps(schema), think_end)

    def json_object(self, think_end: Optional[int] = None) -> Constraint:
        return self._get("json_object", "", think_end)

    def ebnf(self, source: str, think_end: Optional[int] = None) -> Constraint:
        return self._get("ebnf", source, think_end)

    def regex(self, pattern: str, think_end: Optional[int] = None) -> Constraint:
        return self._get("regex", pattern, think_end)

    def tool_call(self, think_end: Optional[int] = None) -> Constraint:
        return self._get("tool_call", TOOL_CALL_EBNF, think_end)

    def recompile(self, kind: str, source: str, think_end: Optional[int] = None) -> Constraint:
        """Rebuilds a constraint from what another rank broadcast."""
        return self._get(kind, source, think_end)

    def state(self, constraint: Constraint) -> "GrammarState":
        return GrammarState(constraint, self.vocab_size)


class GrammarState:
    """One request's position in its grammar."""

    def __init__(self, constraint: Constraint, vocab_size: int):
        self.constraint = constraint
        self.vocab_size = vocab_size
        self.matcher = xgr.GrammarMatcher(constraint.compiled)
        self.armed = constraint.think_end is None
        self.failed = False             # a token outside the grammar was pushed (the mask was not applied upstream)
        self._mask = xgr.allocate_token_bitmask(1, vocab_size)      # int32 [1, words], host

    @property
    def complete(self) -> bool:
        return self.armed and self.matcher.is_terminated()

    def push(self, token: int) -> None:
        if not self.armed:
            if token == self.constraint.think_end:
                self.armed = True
            return
        if self.failed or self.matcher.is_terminated():
            return
        if not self.matcher.accept_token(int(token)):
            self.failed = True

    def mask(self) -> Optional[torch.Tensor]:
        """Allowed tokens now: int32 [words] on the host, or None when nothing is constrained (reasoning, or a
        state that left the grammar)."""
        if not self.armed or self.failed or self.matcher.is_terminated():
            return None
        self.matcher.fill_next_token_bitmask(self._mask, 0)
        return self._mask[0]

    def verify_masks(self, drafted: Sequence[int]) -> list:
        """Masks for the rows of a verify block: row j is chosen after drafted[:j]. Rows after a drafted token the
        grammar refuses get None (acceptance stops there anyway). The matcher ends where it started."""
        out, taken = [], 0
        armed = self.armed
        for j in range(len(drafted) + 1):
            if not armed:
                out.append(None)
            elif self.failed or self.matcher.is_terminated():
                out.append(None)
            else:
                row = xgr.allocate_token_bitmask(1, self.vocab_size)
                self.matcher.fill_next_token_bitmask(row, 0)
                out.append(row[0])
            if j == len(drafted):
                break
            tok = int(drafted[j])
            if not armed:
                armed = tok == self.constraint.think_end
                continue
            if self.matcher.is_terminated() or not self.matcher.accept_token(tok):
                out.extend([None] * (len(drafted) - j))
                break
            taken += 1
        if taken:
            self.matcher.rollback(taken)
        return out


def stack_masks(masks: Sequence[Optional[torch.Tensor]], words: int) -> Optional[torch.Tensor]:
    """[rows, words] int32 for the sampling kernels (all ones where a row is unconstrained); None if none is."""
    if all(m is None for m in masks):
        return None
    out = torch.full((len(masks), words), -1, dtype=torch.int32)
    for i, m in enumerate(masks):
        if m is not None:
            out[i] = m
    return out


def grammars_for(tokenizer, vocab_size: int) -> Grammars:
    """A `Grammars` for one of this package's tokenizers: token i's text as the grammar engine must see it."""
    eos = getattr(tokenizer, "eos_id", None)
    if hasattr(tokenizer, "OFFSET"):            # ByteTokenizer: specials, then the 256 byte values
        off = tokenizer.OFFSET
        vocab = [b"<special%d>" % i for i in range(off)] + [bytes([i]) for i in range(256)]
    else:
        vocab = [tokenizer.decode_bytes([i]) for i in range(tokenizer.vocab_size)]
    vocab += [b"<unused%d>" % i for i in range(len(vocab), vocab_size)]
    return Grammars(vocab[:vocab_size], vocab_size=vocab_size, stop_ids=[eos] if eos is not None else ())


def constraint_from_body(body: dict, grammars: Grammars, think_end: Optional[int] = None) -> Optional[Constraint]:
    """OpenAI `response_format` (json_object / json_schema), SGLang `json_schema` / `regex` / `ebnf`, or a forced
    tool call (`tool_choice` = "required" or a named function) -> a compiled constraint; None when the body asks
    for none. Raises ValueError for a malformed request."""
    rf = body.get("response_format")
    if isinstance(rf, dict):
        kind = rf.get("type")
        if kind == "json_object":
            return grammars.json_object(think_end)
        if kind == "json_schema":
            spec = rf.get("json_schema") or {}
            schema = spec.get("schema", spec)
            if not isinstance(schema, (dict, str)):
                raise ValueError("response_format.json_schema.schema must be an object")
            return grammars.json_schema(schema, think_end)
        if kind not in (None, "text"):
            raise ValueError(f"unknown response_format type {kind!r}")
    if body.get("json_schema") is not None:
        return grammars.json_schema(body["json_schema"], think_end)
    if body.get("regex") is not None:
        return grammars.regex(str(body["regex"]), think_end)
    if body.get("ebnf") is not None:
        return grammars.ebnf(str(body["ebnf"]), think_end)
    choice = body.get("tool_choice")
    if body.get("tools") and (choice == "required" or isinstance(choice, dict)):
        return grammars.tool_call(think_end)
    return None
