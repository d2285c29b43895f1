"""Extracts `<tool_call>{json}</tool_call>` blocks from generated text (reference: hibana/api/parsers/tools.py)."""
from __future__ import annotations

import json
import re
import uuid

_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str) -> tuple[str, list]:
    """Returns (text without the call blocks, OpenAI-style tool_calls)."""
    calls = []
    for m in _CALL.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        name = obj.get("name")
        if not isinstance(name, str):
            continue
        args = obj.get("arguments", obj.get("parameters", {}))
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}})
    return (_CALL.sub("", text).strip() if calls else text), calls
