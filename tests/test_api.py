"""HTTP surface against a real engine loop over the tiny dense model on CPU (httpx ASGI client)."""
import asyncio
import json

import httpx
import pytest
import torch

from hibana_b200.api.messages import to_chat_messages
from hibana_b200.api.parsers.reasoning import ReasoningParser
from hibana_b200.api.parsers.tools import parse_tool_calls
from hibana_b200.api.detok import IncrementalDetok
from hibana_b200.api.server import create_app
from hibana_b200.engine.executor import Executor
from hibana_b200.engine.loop import EngineLoop
from hibana_b200.engine.scheduler import Scheduler, SchedulerConfig
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled
from hibana_b200.tokenizer import ByteTokenizer


@pytest.fixture(scope="module")
def stack():
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    ex = Executor(model, max_batch=4, max_ctx=512, use_graphs=False)
    loop = EngineLoop(Scheduler(ex, SchedulerConfig(max_batch=4, max_queue=8, prefill_chunk=64))).start()
    tok = ByteTokenizer(t.vocab)
    app = create_app(loop, tok, model_name="tiny")
    yield app, loop, tok
    loop.stop()


def _client(app):
    return httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://test")


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


def test_health_models_tokenize_metrics(stack):
    app, loop, tok = stack

    async def go():
        async with _client(app) as c:
            assert (await c.get("/health")).json() == {"status": "ok"}
            assert (await c.get("/v1/models")).json()["data"][0]["id"] == "tiny"
            r = (await c.post("/v1/tokenize", json={"text": "héllo"})).json()
            assert r["count"] == len("héllo".encode()) and tok.decode(r["tokens"]) == "héllo"
            m = (await c.get("/metrics")).text
            assert "hibana_healthy 1" in m
            info = (await c.get("/get_server_info")).json()
            assert info["model"] == "tiny" and "stats" in info
    _run(go())


def test_generate_completions_chat(stack):
    app, loop, tok = stack

    async def go():
        async with _client(app) as c:
            r = await c.post("/generate", json={"text": "abc", "sampling_params": {"max_new_tokens": 5}})
            assert r.status_code == 200 and len(r.json()["output_ids"]) == 5
            r2 = await c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5, "n": 2})
            ch = r2.json()["choices"]
            assert len(ch) == 2 and ch[0]["text"] == ch[1]["text"]          # greedy: identical
            assert r2.json()["usage"]["completion_tokens"] == 10
            r3 = await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                            "max_tokens": 4})
            body = r3.json()
            assert body["choices"][0]["message"]["role"] == "assistant" and body["usage"]["completion_tokens"] == 4
            r4 = await c.post("/v1/chat/completions", json={"messages": [], "max_tokens": 4})
            assert r4.status_code == 400
            r5 = await c.post("/v1/completions", json={"prompt": "x", "max_tokens": 0})
            assert r5.status_code == 400
    _run(go())


def test_streaming_chat_and_anthropic(stack):
    app, loop, tok = stack

    async def go():
        async with _client(app) as c:
            async with c.stream("POST", "/v1/chat/completions", json={
                    "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "stream": True}) as r:
                lines = [l async for l in r.aiter_lines() if l.startswith("data: ")]
            assert lines[-1] == "data: [DONE]"
            chunks = [json.loads(l[6:]) for l in lines[:-1]]
            assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
            assert chunks[-1]["choices"][0]["finish_reason"] == "length"
            r = await c.post("/v1/messages", json={"max_tokens": 5, "system": [{"type": "text", "text": "be brief"}],
                                                   "messages": [{"role": "user", "content": "hello"}]})
            body = r.json()
            assert body["type"] == "message" and body["stop_reason"] == "max_tokens"
            assert body["usage"]["output_tokens"] == 5
            n = (await c.post("/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "hello"}]}
                              )).json()["input_tokens"]
            assert n > 5
            async with c.stream("POST", "/v1/messages", json={"max_tokens": 4, "stream": True, "messages": [
                    {"role": "user", "content": "hello"}]}) as r:
                text = "".join([l async for l in r.aiter_text()])
            assert "event: message_start" in text and "event: message_stop" in text
            assert (await c.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}]})).status_code == 400
    _run(go())


def test_engine_failure_gives_503():
    class Boom:
        def validate_request(self, r): pass
        def can_admit(self, r): return True
        def admit(self, r): raise RuntimeError("device lost")
        def release(self, r): pass
        def retract(self, r): pass
    loop = EngineLoop(Scheduler(Boom(), SchedulerConfig())).start()
    app = create_app(loop, ByteTokenizer())

    async def go():
        async with _client(app) as c:
            r = await c.post("/generate", json={"text": "abc", "sampling_params": {"max_new_tokens": 2}})
            assert r.status_code == 503
            assert (await c.get("/health")).status_code == 503
            r = await c.post("/generate", json={"text": "abc"})
            assert r.status_code == 503
    _run(go())
    loop.stop()


def test_parsers_and_detok():
    rp = ReasoningParser()
    out = [rp.push(p) for p in ("<thi", "nk>plan", " more</th", "ink>answer")]
    r = "".join(o[0] for o in out) + rp.flush()[0]
    c = "".join(o[1] for o in out) + rp.flush()[1]
    assert r == "plan more" and c == "answer"
    text, calls = parse_tool_calls('ok <tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call>')
    assert text == "ok" and calls[0]["function"]["name"] == "f" and json.loads(calls[0]["function"]["arguments"]) == {"a": 1}
    tok = ByteTokenizer()
    d = IncrementalDetok(tok)
    ids = tok.encode("é✓")
    pieces = [d.push([i]) for i in ids]
    assert "".join(pieces) + d.flush() == "é✓" and pieces[0] == ""
    msgs, tools = to_chat_messages({"system": "s", "messages": [
        {"role": "user", "content": [{"type": "text", "text": "q"}]},
        {"role": "assistant", "content": [{"type": "tool_use", "id": "t1", "name": "f", "input": {"x": 1}}]},
        {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "t1", "content": "42"}]}],
        "tools": [{"name": "f", "input_schema": {"type": "object"}}]})
    assert [m["role"] for m in msgs] == ["system", "user", "assistant", "tool"] and tools[0]["function"]["name"] == "f"


def test_constrained_output_over_http(stack):
    """`regex` / `response_format` reach the engine as grammar masks; a malformed schema is a 400."""
    pytest.importorskip("xgrammar")
    import re
    app, loop, tok = stack

    async def go():
        async with _client(app) as c:
            r = await c.post("/generate", json={"text": "go", "sampling_params": {"regex": "(ab|cd){2,3}!",
                                                                                   "max_new_tokens": 24}})
            assert r.status_code == 200, r.text
            assert re.fullmatch(r"(ab|cd){2,3}!", r.json()["text"]), r.json()
            r2 = await c.post("/v1/chat/completions", json={
                "model": "tiny", "messages": [{"role": "user", "content": "json"}], "max_tokens": 48,
                "response_format": {"type": "json_schema", "json_schema": {"schema": {
                    "type": "object", "properties": {"a": {"type": "boolean"}}, "required": ["a"],
                    "additionalProperties": False}}}})
            assert r2.status_code == 200, r2.text
            assert json.loads(r2.json()["choices"][0]["message"]["content"]) in ({"a": True}, {"a": False})
            r3 = await c.post("/generate", json={"text": "x", "sampling_params": {"ebnf": "root ::= ("}})
            assert r3.status_code == 400
    _run(go())


def test_refusal_guard_nudges_then_stops():
    from hibana_b200.api import refusal_guard as rg
    def convo(n):
        msgs = [{"role": "user", "content": "please deploy"}]
        for i in range(n):
            msgs.append({"role": "assistant", "content": "", "tool_calls": [
                {"id": f"c{i}", "type": "function", "function": {"name": "bash", "arguments": "{}"}}]})
            msgs.append({"role": "tool", "tool_call_id": f"c{i}", "content": "This command requires approval"})
        return msgs
    assert rg.decide(convo(1), {})[0] == "generate"
    verdict, found = rg.decide(convo(4), {})
    assert verdict == "nudge" and found.tool == "bash" and found.count == 4
    assert "do not call `bash` again" in rg.reminder(found)["content"]
    assert rg.decide(convo(9), {})[0] == "stop"
    assert rg.decide(convo(9), {"refusal_guard": False})[0] == "generate"
    # a new user message resets the count; ordinary tool errors that differ each time never trigger
    assert rg.decide(convo(9) + [{"role": "user", "content": "try again with sudo"}], {})[0] == "generate"
    varied = [{"role": "user", "content": "x"}] + [
        {"role": "tool", "tool_call_id": str(i), "content": f"error {i}: file not found", "is_error": True} for i in range(9)]
    assert rg.decide(varied, {})[0] == "generate"


def test_chat_stops_without_generating_when_refusals_repeat_and_reports_logprobs():
    from test_scheduler import FakeExecutor
    loop = EngineLoop(Scheduler(FakeExecutor(), SchedulerConfig(max_batch=4))).start()
    app = create_app(loop, ByteTokenizer())
    msgs = [{"role": "user", "content": "go"}]
    for i in range(8):
        msgs.append({"role": "assistant", "content": "", "tool_calls": [
            {"id": f"c{i}", "type": "function", "function": {"name": "write", "arguments": "{}"}}]})
        msgs.append({"role": "tool", "tool_call_id": f"c{i}", "content": "permission denied"})

    async def go():
        async with _client(app) as c:
            r = await c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 4})
            assert r.status_code == 200
            body = r.json()
            assert "`write` was refused 8 times" in body["choices"][0]["message"]["content"]
            assert body["usage"]["completion_tokens"] == 0 and loop.steps == 0
            r = await c.post("/v1/messages", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
            assert r.status_code == 200
    _run(go())
    loop.stop()


def test_image_parts_become_placeholders_or_notes():
    import base64
    from hibana_b200.api import media as m
    from hibana_b200.engine.media import placeholder_ids
    png = base64.b64encode(b"\\x89PNG fake image bytes").decode()
    messages = [{"role": "user", "content": [
        {"type": "text", "text": "what is <image> in this? "},
        {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{png}"}},
        {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": png}}]}]
    assert m.has_images(messages)
    out, plan = m.prepare(messages)
    assert len(plan.images) == 2 and out[0]["content"].count(m.MARKER) == 2      # the user's own "<image>" is escaped
    tok = ByteTokenizer()
    ids = m.expand("A" + out[0]["content"] + "B", tok, plan, tokens_per_image=5)
    neg = [i for i in ids if i < 0]
    assert len(neg) == 10 and neg[:5] == placeholder_ids(plan.images[0], 5) and neg[:5] == neg[5:]   # same bytes
    assert plan.spans[0][1] == 5 and ids[plan.spans[0][0]] < 0 and ids[plan.spans[0][0] - 1] >= 0
    assert "<image>" in tok.decode([i for i in ids if i >= 0])                     # user text survives unescaped
    assert "image omitted" in m.strip_images(messages)[0]["content"]
    import pytest as _pytest
    from hibana_b200.api.validation import BadRequest
    with _pytest.raises(BadRequest):
        m.prepare([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}])
