"""Control clients of a running server: status, cache, stop, verify, chat REPL (HTTP, stdlib only).
Reference: hibana/launch/ctl.py."""
from __future__ import annotations

import json
import os
import signal
import urllib.error
import urllib.request
from pathlib import Path
from typing import Optional


def _url(host: str, port: int, path: str) -> str:
    return f"http://{host}:{port}{path}"


def http_json(host: str, port: int, path: str, body: Optional[dict] = None, timeout: float = 30.0):
    data = json.dumps(body).encode() if body is not None else None
    req = urllib.request.Request(_url(host, port, path), data=data,
                                 headers={"content-type": "application/json"} if data else {})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        raw = r.read().decode()
    try:
        return json.loads(raw)
    except json.JSONDecodeError:
        return raw


def status(host: str, port: int) -> dict:
    try:
        info = http_json(host, port, "/get_server_info", timeout=5)
        return {"running": True, **info}
    except (urllib.error.URLError, OSError) as e:
        return {"running": False, "error": str(e)}


def cache(host: str, port: int, flush: bool = False) -> dict:
    if flush:
        return http_json(host, port, "/flush_cache", {})
    return status(host, port).get("stats", {}).get("cache", {})


def verify(host: str, port: int, prompt: str = "1 + 1 =", max_tokens: int = 8) -> dict:
    """Canary request: same greedy prompt twice must give identical tokens."""
    a = http_json(host, port, "/generate", {"text": prompt, "sampling_params": {"max_new_tokens": max_tokens}})
    b = http_json(host, port, "/generate", {"text": prompt, "sampling_params": {"max_new_tokens": max_tokens}})
    return {"ok": a["output_ids"] == b["output_ids"], "tokens": a["output_ids"],
            "cached_second": b["meta_info"].get("cached_tokens", 0)}


def pid_file(port: int) -> Path:
    root = Path(os.environ.get("HIBANA_RESULTS", str(Path.home() / ".cache" / "hibana")))
    return root / "run" / f"server-{port}.pid"


def stop(port: int) -> bool:
    f = pid_file(port)
    if not f.exists():
        return False
    try:
        os.kill(int(f.read_text().strip()), signal.SIGTERM)
    except (ProcessLookupError, ValueError):
        f.unlink(missing_ok=True)
        return False
    return True


def chat_repl(host: str, port: int, max_tokens: int = 256) -> None:
    messages = []
    while True:
        try:
            line = input("> ")
        except (EOFError, KeyboardInterrupt):
            print()
            return
        if line.strip() in ("/quit", "/exit"):
            return
        if line.strip() == "/reset":
            messages = []
            continue
        messages.append({"role": "user", "content": line})
        r = http_json(host, port, "/v1/chat/completions", {"messages": messages, "max_tokens": max_tokens}, timeout=600)
        text = r["choices"][0]["message"]["content"]
        print(text)
        messages.append({"role": "assistant", "content": text})
