"""Quality / speed tooling on a tiny model: the lossy gate's layers and verdicts, closed-loop streams, evaluation."""
import asyncio
import json

import torch

from hibana_b200 import config as cfgmod
from hibana_b200.api.server import create_app
from hibana_b200.engine.executor import Executor
from hibana_b200.engine.loop import EngineLoop
from hibana_b200.engine.scheduler import Scheduler, SchedulerConfig
from hibana_b200.evals import evaluate, h2h, lossy_gate
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled
from hibana_b200.tokenizer import ByteTokenizer


def test_gate_statistics():
    base = torch.randn(40, 100)
    agree, kl = lossy_gate.distribution_distance(base, base)
    assert agree.mean() == 1.0 and kl.max() < 1e-6
    agree, kl = lossy_gate.distribution_distance(base, base + torch.randn(40, 100))
    assert agree.mean() < 1.0 and kl.mean() > 0.01
    m, lo, hi = lossy_gate.bootstrap_ci([0.1] * 50 + [0.3] * 50)
    assert lo <= m <= hi and abs(m - 0.2) < 1e-9
    assert lossy_gate.mcnemar(0, 0) == 1.0 and lossy_gate.mcnemar(10, 0) < 0.01 and lossy_gate.mcnemar(5, 5) > 0.5
    ps = lossy_gate.frozen_prompts(1000)
    assert len(ps) == 24 and ps == lossy_gate.frozen_prompts(1000) and {p["domain"] for p in ps} == set(lossy_gate.DOMAINS)
    assert lossy_gate.score_item("the answer is 42", {"answer": "42"}) and not lossy_gate.score_item("41", {"answer": "42", "scorer": "exact"})


def test_gate_verdicts_on_a_tiny_model(tmp_path):
    t = scaled(dense_tiny(), weight_format="bf16")
    good = DenseModel(t, "cpu", seed=0)
    noisy = DenseModel(t, "cpu", seed=0)
    for layer in noisy.layers:                              # a "lossy option": perturbed MLP weights
        layer.down.weight += torch.randn_like(layer.down.weight.float()).to(torch.bfloat16) * 0.05
    cfg = cfgmod.EngineConfig(target="dense-tiny", max_batch=8, cuda_graphs=False)

    def maker(model):
        return lambda c: Executor(model, max_batch=8, max_ctx=256, use_graphs=False)
    same = lossy_gate.run_gate(maker(good), cfg, cfg, t.vocab, tmp_path / "same", continuation=8)
    assert same["verdict"] == "exact" and all(d["within_floor"] for d in same["layer1"].values())
    assert (tmp_path / "same" / "scorecard.json").exists()
    built = iter([good, noisy])
    lossy = lossy_gate.run_gate(lambda c: Executor(next(built), max_batch=8, max_ctx=256, use_graphs=False), cfg, cfg,
                                t.vocab, tmp_path / "lossy", continuation=8, min_gain=100.0)
    assert lossy["verdict"] == "reject"                   # measurably different and not faster
    assert any(not d["within_floor"] for d in lossy["layer1"].values())


def _app():
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_scheduler import FakeExecutor
    loop = EngineLoop(Scheduler(FakeExecutor(), SchedulerConfig(max_batch=8))).start()
    return loop, create_app(loop, ByteTokenizer())


def test_streams_and_evaluate(tmp_path):
    import httpx
    loop, app = _app()

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t", timeout=60) as c:
            async def post(body):
                return (await c.post("/generate", json=body)).json()
            await post({"input_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 2}})   # first request pays lazy imports
            r = await h2h.run_streams(post, 3, duration_s=0.4, warmup_s=0.1, prompt_tokens=8, max_tokens=4)
            assert r["requests"] >= 3 and r["aggregate_tok_s"] > 0
            res = await h2h.head_to_head(post, post, [1, 2], duration_s=0.2, warmup_s=0.05, prompt_tokens=8, max_tokens=4)
            table = h2h.markdown(res)
            assert table.count("\n") == 3 and "| 2 |" in table
        tasks = [{"prompt": "abc", "answer": "", "scorer": "contains", "max_tokens": 4},
                 {"messages": [{"role": "user", "content": "hi"}], "answer": "zzz-never", "max_tokens": 4}]
        cfg = cfgmod.EngineConfig(target="dense-tiny")
        out = await evaluate.evaluate(app, cfg, tasks, tmp_path / "ev", speed=True, streams=(1,))
        assert out["suite"]["items"] == 2 and out["suite"]["correct"] == 1
        assert (tmp_path / "ev" / "SUMMARY.md").read_text().startswith("# Evaluation summary")
        assert json.loads((tmp_path / "ev" / "manifest.json").read_text())["config"]["target"] == "dense-tiny"
        again = await evaluate.evaluate(app, cfg, tasks, tmp_path / "ev")      # resumes: nothing is re-run
        assert again["suite"]["correct"] == 1
        assert len((tmp_path / "ev" / "suite" / "results.jsonl").read_text().splitlines()) == 2
    asyncio.run(go())
    loop.stop()
