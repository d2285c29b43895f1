"""Chat template rendering (jinja2). Default is ChatML; a checkpoint's own template is used when present.
Reference: hibana/api/chat_template.py."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import jinja2

CHATML = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
    "{% if m['content'] is string %}{{ m['content'] }}{% else %}{% for p in m['content'] %}"
    "{% if p['type'] == 'text' %}{{ p['text'] }}{% elif p['type'] == 'image' %}<image>{% endif %}{% endfor %}{% endif %}"
    "{% if m.get('tool_calls') %}{% for c in m['tool_calls'] %}\n<tool_call>\n{{ c['function'] | tojson }}\n</tool_call>"
    "{% endfor %}{% endif %}<|im_end|>\n{% endfor %}"
    "{% if tools %}{# tools are described in the system turn by the caller #}{% endif %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% if enable_thinking is defined and not enable_thinking %}"
    "<think>\n\n</think>\n\n{% endif %}{% endif %}")


class ChatTemplate:
    def __init__(self, source: Optional[str] = None):
        env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False)
        env.filters["tojson"] = lambda v: json.dumps(v, ensure_ascii=False)
        self.template = env.from_string(source or CHATML)

    @classmethod
    def load(cls, checkpoint: Optional[str]) -> "ChatTemplate":
        if checkpoint:
            cfg = Path(checkpoint) / "tokenizer_config.json"
            if cfg.exists():
                src = json.loads(cfg.read_text()).get("chat_template")
                if isinstance(src, str):
                    return cls(src)
        return cls()

    def render(self, messages: list, tools: Optional[list] = None, add_generation_prompt: bool = True, **kw) -> str:
        msgs = list(messages)
        if tools:
            desc = "You may call these tools by emitting <tool_call>{\"name\": ..., \"arguments\": {...}}</tool_call>:\n" + \
                   "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
            if msgs and msgs[0]["role"] == "system" and isinstance(msgs[0]["content"], str):
                msgs[0] = dict(msgs[0], content=msgs[0]["content"] + "\n\n" + desc)
            else:
                msgs.insert(0, {"role": "system", "content": desc})
        return self.template.render(messages=msgs, tools=tools, add_generation_prompt=add_generation_prompt, **kw)
