"""Refusal guard: keeps an agent from hammering a tool its harness keeps refusing.

Agent harnesses answer a tool call they will not run with a short error result ("requires approval", "permission
denied"). Some models respond by retrying the same call with small variations, hundreds of times. Every request
carries the whole conversation, so the server can see this without keeping state: it counts, since the last real
user message, tool results that (a) are marked as errors or read like a permission refusal and (b) repeat word for
word for the same tool. From `NUDGE` repeats on a reminder is appended to the conversation before it is rendered;
from `STOP` repeats on the server answers by itself with a short explanation and generates nothing. A request
opts out with `"refusal_guard": false`. Reference: hibana/api/refusal_guard.py:1-100.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Optional

NUDGE, STOP = 3, 8
MAX_REFUSAL_CHARS = 400
_WORDS = re.compile(r"requires? approval|permission|denied|not allowed|not permitted|rejected|refused|blocked", re.I)


@dataclass(frozen=True)
class Repeated:
    tool: str
    text: str
    count: int


def _plain(content) -> str:
    if isinstance(content, str):
        return content
    if isinstance(content, list):
        return "".join(p.get("text", "") for p in content if isinstance(p, dict))
    return ""


def _from_user(msg: dict) -> bool:
    if msg.get("role") != "user":
        return False
    text = _plain(msg.get("content")).strip()
    harness_note = text.startswith("<system-reminder>") and text.endswith("</system-reminder>")
    return bool(text) and not harness_note


def find_repeated(messages: list) -> Optional[Repeated]:
    """The most frequent (tool, refusal text) pair among tool results after the last user message, if it occurs at
    least twice."""
    last_user = max((i for i, m in enumerate(messages) if isinstance(m, dict) and _from_user(m)), default=0)
    call_names: dict = {}
    tally: dict = {}
    for m in messages[last_user:]:
        if not isinstance(m, dict):
            continue
        for call in m.get("tool_calls") or []:
            if isinstance(call, dict):
                call_names[call.get("id")] = (call.get("function") or {}).get("name", "")
        if m.get("role") != "tool":
            continue
        text = _plain(m.get("content")).strip()
        if not text or len(text) > MAX_REFUSAL_CHARS:
            continue
        if not (m.get("is_error") or _WORDS.search(text)):
            continue
        key = (call_names.get(m.get("tool_call_id"), ""), text)
        tally[key] = tally.get(key, 0) + 1
    if not tally:
        return None
    (tool, text), n = max(tally.items(), key=lambda kv: kv[1])
    return Repeated(tool, text, n) if n >= 2 else None


def reminder(r: Repeated) -> dict:
    name = f"`{r.tool}`" if r.tool else "that tool"
    return {"role": "user", "content": (
        f"<system-reminder>\n{name} has now been refused {r.count} times with \"{r.text[:200]}\". Another attempt "
        f"will be refused as well: do not call {name} again. Finish what can be done without it and tell the user "
        f"which permission or change is needed.\n</system-reminder>")}


def stop_text(r: Repeated) -> str:
    name = f"`{r.tool}`" if r.tool else "a tool"
    return (f"I am stopping here: {name} was refused {r.count} times (\"{r.text[:200]}\"), so this step cannot go on. "
            f"Please grant the permission or run it yourself, then tell me how to continue.")


def decide(messages: list, body: dict) -> tuple[str, Optional[Repeated]]:
    """("generate" | "nudge" | "stop", what was found)."""
    if body.get("refusal_guard") is False:
        return "generate", None
    r = find_repeated(messages)
    if r is None or r.count < NUDGE:
        return "generate", r
    return ("stop" if r.count >= STOP else "nudge"), r
