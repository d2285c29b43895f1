"""Anthropic Messages API <-> internal chat messages, and the SSE event writer for streamed replies.
Reference: hibana/api/messages.py:1-374."""
from __future__ import annotations

import json
import uuid
from typing import Iterable, Optional


def to_chat_messages(body: dict) -> tuple[list, Optional[list]]:
    """Anthropic request body -> (OpenAI-style messages, tools)."""
    msgs: list = []
    system = body.get("system")
    if isinstance(system, list):
        system = "\n".join(b.get("text", "") for b in system if b.get("type") == "text")
    if system:
        msgs.append({"role": "system", "content": system})
    for m in body.get("messages", []):
        role, content = m.get("role"), m.get("content")
        if isinstance(content, str):
            msgs.append({"role": role, "content": content})
            continue
        text_parts, tool_calls = [], []
        for block in content or []:
            kind = block.get("type")
            if kind == "text":
                text_parts.append({"type": "text", "text": block.get("text", "")})
            elif kind == "image":
                text_parts.append({"type": "image", "source": block.get("source")})
            elif kind == "thinking":
                continue
            elif kind == "tool_use":
                tool_calls.append({"id": block.get("id"), "type": "function",
                                   "function": {"name": block.get("name"), "arguments": block.get("input", {})}})
            elif kind == "tool_result":
                res = block.get("content")
                if isinstance(res, list):
                    res = "\n".join(b.get("text", "") for b in res if b.get("type") == "text")
                msgs.append({"role": "tool", "tool_call_id": block.get("tool_use_id"), "content": res or ""})
        if text_parts or tool_calls:
            entry = {"role": role, "content": text_parts if len(text_parts) != 1 or text_parts[0]["type"] != "text"
                     else text_parts[0]["text"]}
            if not text_parts:
                entry["content"] = ""
            if tool_calls:
                entry["tool_calls"] = tool_calls
            msgs.append(entry)
    tools = None
    if body.get("tools"):
        tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                   "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    return msgs, tools


def message_response(model: str, text: str, reasoning: str, tool_calls: list, stop_reason: str, usage: dict) -> dict:
    content = []
    if reasoning:
        content.append({"type": "thinking", "thinking": reasoning, "signature": ""})
    if text:
        content.append({"type": "text", "text": text})
    for c in tool_calls:
        args = c["function"]["arguments"]
        content.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["function"]["name"],
                        "input": json.loads(args) if isinstance(args, str) else args})
    return {"id": "msg_" + uuid.uuid4().hex[:24], "type": "message", "role": "assistant", "model": model,
            "content": content, "stop_reason": "tool_use" if tool_calls else stop_reason, "stop_sequence": None,
            "usage": usage}


def stop_reason(finish: Optional[str]) -> str:
    return {"stop": "end_turn", "length": "max_tokens", "cancelled": "end_turn"}.get(finish or "stop", "end_turn")


class EventWriter:
    """Builds the Anthropic SSE sequence: message_start, content_block_start/delta/stop, message_delta, message_stop."""

    def __init__(self, model: str, input_tokens: int):
        self.model, self.input_tokens = model, input_tokens
        self.index = -1
        self.open_kind: Optional[str] = None
        self.mid = "msg_" + uuid.uuid4().hex[:24]

    @staticmethod
    def _sse(event: str, data: dict) -> str:
        return f"event: {event}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n"

    def start(self) -> str:
        return self._sse("message_start", {"type": "message_start", "message": {
            "id": self.mid, "type": "message", "role": "assistant", "model": self.model, "content": [],
            "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": self.input_tokens, "output_tokens": 0}}})

    def _open(self, kind: str) -> str:
        out = self.close_block()
        self.index += 1
        self.open_kind = kind
        block = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
        return out + self._sse("content_block_start", {"type": "content_block_start", "index": self.index,
                                                       "content_block": block})

    def close_block(self) -> str:
        if self.open_kind is None:
            return ""
        self.open_kind = None
        return self._sse("content_block_stop", {"type": "content_block_stop", "index": self.index})

    def delta(self, kind: str, text: str) -> str:
        if not text:
            return ""
        out = self._open(kind) if self.open_kind != kind else ""
        d = {"type": "thinking_delta", "thinking": text} if kind == "thinking" else {"type": "text_delta", "text": text}
        return out + self._sse("content_block_delta", {"type": "content_block_delta", "index": self.index, "delta": d})

    def tool_use(self, call: dict) -> str:
        out = self.close_block()
        self.index += 1
        args = call["function"]["arguments"]
        out += self._sse("content_block_start", {"type": "content_block_start", "index": self.index, "content_block": {
            "type": "tool_use", "id": call["id"].replace("call_", "toolu_"), "name": call["function"]["name"], "input": {}}})
        out += self._sse("content_block_delta", {"type": "content_block_delta", "index": self.index, "delta": {
            "type": "input_json_delta", "partial_json": args if isinstance(args, str) else json.dumps(args)}})
        return out + self._sse("content_block_stop", {"type": "content_block_stop", "index": self.index})

    def finish(self, reason: str, output_tokens: int) -> str:
        out = self.close_block()
        out += self._sse("message_delta", {"type": "message_delta", "delta": {"stop_reason": reason,
                                                                               "stop_sequence": None},
                                           "usage": {"output_tokens": output_tokens}})
        return out + self._sse("message_stop", {"type": "message_stop"})

    def error(self, message: str) -> str:
        return self._sse("error", {"type": "error", "error": {"type": "api_error", "message": message}})
