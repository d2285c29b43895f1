"""Request validation: JSON bodies -> SamplingParams (reference: hibana/api/validation.py)."""
from __future__ import annotations

from typing import Optional

from ..engine.request import SamplingParams


class BadRequest(ValueError):
    pass


def _num(body: dict, key: str, default, lo=None, hi=None, kind=float):
    v = body.get(key, default)
    if v is None:
        return default
    try:
        v = kind(v)
    except (TypeError, ValueError):
        raise BadRequest(f"{key} must be a number") from None
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise BadRequest(f"{key} out of range")
    return v


def sampling_from(body: dict, tokenizer=None, default_max: int = 256, max_limit: int = 1 << 20,
                  grammars=None) -> SamplingParams:
    """Accepts OpenAI names (max_tokens / max_completion_tokens, stop) and SGLang names (max_new_tokens,
    stop_token_ids) plus the engine's acceptance knobs."""
    max_tokens = body.get("max_tokens", body.get("max_completion_tokens", body.get("max_new_tokens", default_max)))
    max_tokens = _num({"m": max_tokens}, "m", default_max, 1, max_limit, int)
    stop_ids = list(body.get("stop_token_ids") or [])
    stops = body.get("stop")
    if isinstance(stops, str):
        stops = [stops]
    if stops and tokenizer is not None:
        for s in stops:
            ids = tokenizer.encode(s)
            if len(ids) == 1:
                stop_ids.append(ids[0])
    temperature = _num(body, "temperature", 0.0 if body.get("greedy") else body.get("temperature", 0.0), 0.0, 100.0)
    seed = body.get("seed")
    if seed is not None:
        seed = _num(body, "seed", None, 0, (1 << 63) - 1, int)
    constraint = None
    if grammars is not None:       # callable: builds the (cached) engine.grammar.Grammars on first use
        from ..engine.grammar import constraint_from_body
        wants = any(body.get(k) is not None for k in ("response_format", "json_schema", "regex", "ebnf")) or (
            body.get("tools") and body.get("tool_choice") not in (None, "auto", "none"))
        if wants:
            try:
                constraint = constraint_from_body(body, grammars() if callable(grammars) else grammars)
            except Exception as e:     # malformed schema / grammar text
                raise BadRequest(f"invalid output constraint: {e}") from None
    try:
        return SamplingParams(
            constraint=constraint,
            temperature=temperature, top_k=_num(body, "top_k", 0, -1, 1 << 20, int) if body.get("top_k", 0) != -1 else 0,
            top_p=_num(body, "top_p", 1.0, 1e-6, 1.0), max_tokens=max_tokens, stop_ids=tuple(int(i) for i in stop_ids),
            ignore_eos=bool(body.get("ignore_eos", False)), seed=seed,
            accept_top_k=_num(body, "accept_top_k", 1, 1, 64, int), accept_margin=_num(body, "accept_margin", 0.0, 0.0),
            accept_soft=_num(body, "accept_soft", 0.0, 0.0), logprobs=_num(body, "logprobs", 0, 0, 20, int)
            if not isinstance(body.get("logprobs"), bool) else 0)
    except ValueError as e:
        raise BadRequest(str(e)) from None
