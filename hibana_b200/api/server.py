"""HTTP API: OpenAI-compatible (/v1/chat/completions, /v1/completions, /v1/models), Anthropic-compatible
(/v1/messages, /v1/messages/count_tokens), SGLang-style /generate, and operations endpoints (/health, /ready,
/get_server_info, /describe, /metrics, /flush_cache, /v1/tokenize).

`create_app(engine, tokenizer, ...)` builds the FastAPI app around an EngineLoop; HTTP threads only enqueue work and
read ticket events. Status codes: 400 invalid request, 429 queue full, 503 engine unavailable.
Reference: hibana/api/server.py:61-906, docs/api.md:9-21.
"""
from __future__ import annotations

import asyncio
import json
import queue
import time
import uuid
from typing import AsyncIterator, Optional

from fastapi import FastAPI, Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine.loop import EngineLoop, EngineUnavailable, Ticket
from ..engine.scheduler import QueueFull
from . import media as media_api
from . import refusal_guard
from .chat_template import ChatTemplate
from .detok import IncrementalDetok
from .messages import EventWriter, message_response, stop_reason, to_chat_messages
from .parsers.reasoning import ReasoningParser
from .parsers.tools import parse_tool_calls
from .validation import BadRequest, sampling_from


def _err(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": message, "type": kind, "code": status}}, status_code=status)


async def _events(ticket: Ticket) -> AsyncIterator[tuple]:
    """Yields ticket events on the asyncio side; the engine thread wakes us through call_soon_threadsafe."""
    loop = asyncio.get_running_loop()
    wake = asyncio.Event()
    ticket.notify = lambda: loop.call_soon_threadsafe(wake.set)
    while True:
        try:
            item = ticket.events.get_nowait()
        except queue.Empty:
            wake.clear()
            try:
                await asyncio.wait_for(wake.wait(), timeout=0.05)
            except asyncio.TimeoutError:
                pass
            continue
        yield item
        if item[0] in ("done", "error"):
            return


def create_app(engine: EngineLoop, tokenizer, *, model_name: str = "hibana-b200", template: Optional[ChatTemplate] = None,
               info: Optional[dict] = None, api_key: str = "") -> FastAPI:
    app = FastAPI(title="hibana-b200")
    template = template or ChatTemplate()
    info = info or {}
    eos_id = getattr(tokenizer, "eos_id", None)
    _gr: dict = {}

    def grammars():
        """Grammar compiler for this tokenizer, built on the first constrained request."""
        if "g" not in _gr:
            from ..engine.grammar import grammars_for
            _gr["g"] = grammars_for(tokenizer, getattr(engine, "vocab", None) or tokenizer.vocab_size)
        return _gr["g"]

    def _submit(prompt_ids, params, media=None) -> Ticket:
        return engine.submit(prompt_ids, params, eos_id=eos_id, media=media)

    def _vision():
        """The served model's vision encoder (None: the target takes no images)."""
        ex = getattr(getattr(engine, "sched", None), "ex", None)
        return getattr(getattr(ex, "model", None), "vision", None)

    def _guard(fn):
        async def wrapped(req: HttpRequest):
            if api_key and req.headers.get("authorization", "") != f"Bearer {api_key}" and \
                    req.headers.get("x-api-key", "") != api_key:
                return _err(401, "invalid api key", "authentication_error")
            try:
                body = await req.json() if req.method == "POST" else {}
                if not isinstance(body, dict):
                    raise BadRequest("body must be a JSON object")
                return await fn(req, body)
            except BadRequest as e:
                return _err(400, str(e))
            except json.JSONDecodeError:
                return _err(400, "invalid JSON")
            except QueueFull:
                return _err(429, "queue full", "rate_limit_error")
            except EngineUnavailable as e:
                return _err(503, str(e), "service_unavailable")
        return wrapped

    async def _collect(ticket: Ticket, request: Optional[HttpRequest] = None):
        ids, finish = [], None
        async for kind, val in _events(ticket):
            if kind == "tokens":
                ids.extend(val)
            elif kind == "done":
                finish = val
            else:
                raise EngineUnavailable(val) if "queue" not in str(val) else BadRequest(val)
            if request is not None and await request.is_disconnected():
                engine.cancel(ticket)
        return ids, finish

    def _strip_stop(ids, params):
        return ids[:-1] if ids and (ids[-1] in params.stop_ids or ids[-1] == eos_id) else ids

    # ---- operations
    @app.get("/health")
    async def health():
        return JSONResponse({"status": "ok"}) if engine.healthy else _err(503, engine.failure or "engine failed",
                                                                          "service_unavailable")

    @app.get("/ready")
    async def ready():
        return await health()

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "hibana-b200",
                                            "created": int(time.time())}]}

    @app.get("/get_server_info")
    async def server_info():
        return {"model": model_name, **info, "stats": engine.stats()}

    @app.get("/describe")
    async def describe():
        return await server_info()

    @app.get("/metrics")
    async def metrics():
        lines = []
        def walk(prefix, obj):
            for k, v in obj.items():
                if isinstance(v, dict):
                    walk(f"{prefix}{k}_", v)
                elif isinstance(v, bool):
                    lines.append(f"hibana_{prefix}{k} {int(v)}")
                elif isinstance(v, (int, float)) and v is not None:
                    lines.append(f"hibana_{prefix}{k} {v}")
        walk("", engine.stats())
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/flush_cache")
    async def flush_cache():
        state = getattr(engine.sched.ex, "state", None)
        freed = state.cache.flush() if state is not None and state.cache is not None and engine.sched.idle() else 0
        return {"flushed_tokens": freed}

    async def tokenize(req, body):
        text = body.get("text", body.get("prompt", ""))
        ids = tokenizer.encode(text)
        return {"tokens": ids, "count": len(ids)}
    app.post("/v1/tokenize")(_guard(tokenize))
    app.post("/tokenize")(_guard(tokenize))

    # ---- SGLang-style generate
    async def generate(req, body):
        sp_body = dict(body.get("sampling_params") or {})
        params = sampling_from(sp_body, tokenizer, grammars=grammars)
        ids = body.get("input_ids")
        if ids is None:
            if "text" not in body:
                raise BadRequest("text or input_ids required")
            ids = tokenizer.encode(body["text"])
        ticket = _submit(ids, params)
        if body.get("stream"):
            async def gen():
                detok, n = IncrementalDetok(tokenizer), 0
                async for kind, val in _events(ticket):
                    if kind == "tokens":
                        n += len(val)
                        yield f"data: {json.dumps({'text': detok.push(val), 'token_ids': val})}\n\n"
                    elif kind == "error":
                        yield f"data: {json.dumps({'error': val})}\n\n"
                    else:
                        yield f"data: {json.dumps({'text': detok.flush(), 'meta_info': {'finish_reason': val, 'completion_tokens': n}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        out, finish = await _collect(ticket, req)
        return {"text": tokenizer.decode(_strip_stop(out, params)), "output_ids": out,
                "meta_info": {"finish_reason": finish, "prompt_tokens": len(ids), "completion_tokens": len(out),
                              "cached_tokens": getattr(ticket.request, "cached_len", 0)}}
    app.post("/generate")(_guard(generate))

    # ---- OpenAI completions
    async def completions(req, body):
        prompt = body.get("prompt")
        if prompt is None:
            raise BadRequest("prompt required")
        params = sampling_from(body, tokenizer, grammars=grammars)
        ids = prompt if isinstance(prompt, list) and prompt and isinstance(prompt[0], int) else tokenizer.encode(
            prompt if isinstance(prompt, str) else "".join(prompt))
        n = int(body.get("n", 1))
        if n < 1 or n > 16:
            raise BadRequest("n out of range")
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        tickets = [_submit(ids, params) for _ in range(n)]
        if body.get("stream"):
            async def gen():
                for i, t in enumerate(tickets):
                    detok = IncrementalDetok(tokenizer)
                    async for kind, val in _events(t):
                        if kind == "tokens":
                            chunk = {"id": cid, "object": "text_completion", "model": model_name,
                                     "choices": [{"index": i, "text": detok.push(val), "finish_reason": None}]}
                        elif kind == "done":
                            chunk = {"id": cid, "object": "text_completion", "model": model_name,
                                     "choices": [{"index": i, "text": detok.flush(), "finish_reason": val}]}
                        else:
                            chunk = {"error": {"message": val, "type": "service_unavailable"}}
                        yield f"data: {json.dumps(chunk)}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        choices, total = [], 0
        for i, t in enumerate(tickets):
            out, finish = await _collect(t, req)
            total += len(out)
            choices.append({"index": i, "text": tokenizer.decode(_strip_stop(out, params)), "finish_reason": finish})
        return {"id": cid, "object": "text_completion", "model": model_name, "choices": choices,
                "usage": {"prompt_tokens": len(ids), "completion_tokens": total, "total_tokens": len(ids) + total}}
    app.post("/v1/completions")(_guard(completions))

    # ---- OpenAI chat
    def _render(body, messages, tools):
        """(prompt ids, template kwargs, media plan or None). Image parts become placeholder ids when the target has
        a vision encoder, a short note otherwise."""
        kwargs = dict(body.get("chat_template_kwargs") or {})
        plan = None
        if media_api.has_images(messages):
            vision = _vision()
            if vision is None:
                messages = media_api.strip_images(messages)
            else:
                messages, plan = media_api.prepare(messages)
        text = template.render(messages, tools=tools, add_generation_prompt=True, **kwargs)
        if plan is not None and plan.images:
            return media_api.expand(text, tokenizer, plan, _vision().cfg.tokens_per_image), kwargs, plan
        return tokenizer.encode(media_api.unescape(text)), kwargs, None

    def _guarded(body, messages):
        """Refusal guard: ("generate" | "stop", messages (with a reminder appended on a nudge), canned text)."""
        verdict, found = refusal_guard.decide(messages, body)
        if verdict == "nudge":
            return "generate", messages + [refusal_guard.reminder(found)], None
        if verdict == "stop":
            return "stop", messages, refusal_guard.stop_text(found)
        return "generate", messages, None

    def _logprob_entries(ticket, out_ids):
        """OpenAI `logprobs.content` entries for the sampled tokens (the engine records them per token when the
        request asked for them)."""
        lps = getattr(ticket.request, "token_logprobs", None) or []
        entries = []
        for i, tid in enumerate(out_ids):
            rec = lps[i] if i < len(lps) else None
            tok = tokenizer.decode([tid])
            e = {"token": tok, "logprob": rec[0] if rec else None, "bytes": list(tok.encode("utf-8"))}
            e["top_logprobs"] = [{"token": tokenizer.decode([t]), "logprob": lp, "bytes": list(tokenizer.decode([t]).encode("utf-8"))}
                                 for t, lp in (rec[1] if rec else [])]
            entries.append(e)
        return entries

    def _split(text: str, thinking: bool):
        rp = ReasoningParser(starts_in_reasoning=False)
        r1, c1 = rp.push(text)
        r2, c2 = rp.flush()
        content, calls = parse_tool_calls(c1 + c2)
        return r1 + r2, content, calls

    async def chat(req, body):
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            raise BadRequest("messages required")
        if body.get("logprobs") is True:             # OpenAI chat form: logprobs: true + top_logprobs: k
            body = dict(body, logprobs=max(int(body.get("top_logprobs") or 0), 1))
        params = sampling_from(body, tokenizer, grammars=grammars)
        tools = body.get("tools")
        verdict, messages, canned = _guarded(body, messages)
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        if verdict == "stop":      # the harness refused the same call again and again: answer without generating
            if body.get("stream"):
                async def stopped():
                    chunk = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                             "choices": [{"index": 0, "delta": {"role": "assistant", "content": canned},
                                          "finish_reason": "stop"}]}
                    yield f"data: {json.dumps(chunk)}\n\n"
                    yield "data: [DONE]\n\n"
                return StreamingResponse(stopped(), media_type="text/event-stream")
            return {"id": cid, "object": "chat.completion", "created": created, "model": model_name,
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": canned},
                                 "finish_reason": "stop"}],
                    "usage": {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}}
        ids, kwargs, plan = _render(body, messages, tools)
        n = int(body.get("n", 1))
        if n < 1 or n > 16:
            raise BadRequest("n out of range")
        tickets = [_submit(ids, params, plan) for _ in range(n)]
        if body.get("stream"):
            async def gen():
                for i, t in enumerate(tickets):
                    detok, rp, full = IncrementalDetok(tokenizer), ReasoningParser(), ""
                    first = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                             "choices": [{"index": i, "delta": {"role": "assistant", "content": ""},
                                          "finish_reason": None}]}
                    yield f"data: {json.dumps(first)}\n\n"
                    async for kind, val in _events(t):
                        if kind == "error":
                            yield f"data: {json.dumps({'error': {'message': val, 'type': 'service_unavailable'}})}\n\n"
                            continue
                        text = detok.push(val) if kind == "tokens" else detok.flush()
                        r, c = rp.push(text)
                        if kind == "done":
                            r2, c2 = rp.flush()
                            r, c = r + r2, c + c2
                        full += c
                        delta = {}
                        if r:
                            delta["reasoning_content"] = r
                        if c and not tools:
                            delta["content"] = c
                        finish = None
                        if kind == "done":
                            finish = val
                            if tools:
                                content, calls = parse_tool_calls(full)
                                if content:
                                    delta["content"] = content
                                if calls:
                                    delta["tool_calls"] = [dict(c_, index=j) for j, c_ in enumerate(calls)]
                                    finish = "tool_calls"
                        if delta or finish:
                            chunk = {"id": cid, "object": "chat.completion.chunk", "created": created,
                                     "model": model_name,
                                     "choices": [{"index": i, "delta": delta, "finish_reason": finish}]}
                            yield f"data: {json.dumps(chunk, ensure_ascii=False)}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        choices, total = [], 0
        for i, t in enumerate(tickets):
            out, finish = await _collect(t, req)
            total += len(out)
            reasoning, content, calls = _split(tokenizer.decode(_strip_stop(out, params)), True)
            msg = {"role": "assistant", "content": content}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                msg["tool_calls"] = calls
                finish = "tool_calls"
            choice = {"index": i, "message": msg, "finish_reason": finish}
            if params.logprobs:
                choice["logprobs"] = {"content": _logprob_entries(t, _strip_stop(out, params))}
            choices.append(choice)
        return {"id": cid, "object": "chat.completion", "created": created, "model": model_name, "choices": choices,
                "usage": {"prompt_tokens": len(ids), "completion_tokens": total, "total_tokens": len(ids) + total}}
    app.post("/v1/chat/completions")(_guard(chat))

    # ---- Anthropic messages
    async def count_tokens(req, body):
        messages, tools = to_chat_messages(body)
        ids, _, _ = _render(body, messages, tools)
        return {"input_tokens": len(ids)}
    app.post("/v1/messages/count_tokens")(_guard(count_tokens))

    async def anthropic_messages(req, body):
        if "max_tokens" not in body:
            raise BadRequest("max_tokens required")
        messages, tools = to_chat_messages(body)
        if not messages:
            raise BadRequest("messages required")
        b2 = dict(body)
        if "stop_sequences" in body:
            b2["stop"] = body["stop_sequences"]
        params = sampling_from(b2, tokenizer, grammars=grammars)
        verdict, messages, canned = _guarded(body, messages)
        if verdict == "stop":
            if body.get("stream"):
                async def stopped():
                    ew = EventWriter(model_name, 0)
                    yield ew.start()
                    yield ew.delta("text", canned)
                    yield ew.finish("end_turn", 0)
                return StreamingResponse(stopped(), media_type="text/event-stream")
            return message_response(model_name, canned, "", [], "end_turn", {"input_tokens": 0, "output_tokens": 0})
        ids, _, plan = _render(body, messages, tools)
        ticket = _submit(ids, params, plan)
        if body.get("stream"):
            async def gen():
                ew, detok, rp, full, n = EventWriter(model_name, len(ids)), IncrementalDetok(tokenizer), \
                    ReasoningParser(), "", 0
                yield ew.start()
                async for kind, val in _events(ticket):
                    if kind == "error":
                        yield ew.error(val)
                        return
                    if kind == "tokens":
                        n += len(val)
                    text = detok.push(val) if kind == "tokens" else detok.flush()
                    r, c = rp.push(text)
                    if kind == "done":
                        r2, c2 = rp.flush()
                        r, c = r + r2, c + c2
                    full += c
                    yield ew.delta("thinking", r)
                    if not tools:
                        yield ew.delta("text", c)
                    if kind == "done":
                        reason = stop_reason(val)
                        if tools:
                            content, calls = parse_tool_calls(full)
                            yield ew.delta("text", content)
                            for call in calls:
                                yield ew.tool_use(call)
                            if calls:
                                reason = "tool_use"
                        yield ew.finish(reason, n)
            return StreamingResponse(gen(), media_type="text/event-stream")
        out, finish = await _collect(ticket, req)
        reasoning, content, calls = _split(tokenizer.decode(_strip_stop(out, params)), True)
        return message_response(model_name, content, reasoning, calls, stop_reason(finish),
                                {"input_tokens": len(ids), "output_tokens": len(out)})
    app.post("/v1/messages")(_guard(anthropic_messages))

    return app


def serve(cfg=None, *, host: Optional[str] = None, port: Optional[int] = None) -> None:
    """Builds the engine from the current settings and serves it with uvicorn (blocking)."""
    import signal

    import uvicorn

    from .. import config as cfgmod
    from ..engine.llm import LLM
    from ..tokenizer import load_tokenizer

    cfg = cfg or cfgmod.current()
    llm = LLM(cfg, warmup=True)      # checkpoint, memory plan, SSD tier, speculation, graphs: all from the settings
    ckpt = cfg.weights if cfg.weights != "random" else None
    tok = load_tokenizer(ckpt, llm.target.vocab)
    engine = EngineLoop(llm.scheduler).start()
    if cfg.trace_dir:
        from ..engine.traces import TraceSink
        llm.scheduler.sink = TraceSink(cfg.trace_dir, cap_bytes=int(cfg.trace_cap_gb * (1 << 30)))
    app = create_app(engine, tok, model_name=llm.target.name, template=ChatTemplate.load(ckpt),
                     info={"config": cfg.as_dict(), "target": llm.target.name}, api_key=cfg.api_key)
    server = uvicorn.Server(uvicorn.Config(app, host=host or cfg.host, port=port or cfg.port, log_level="warning"))

    def _term(*_):
        engine.drain(30.0)
        server.should_exit = True
    signal.signal(signal.SIGTERM, _term)
    server.run()
    engine.stop()
    llm.shutdown()                   # cached prefixes go to the SSD tier before the process leaves
