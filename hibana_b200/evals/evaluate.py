"""Evaluate one build: serve it in process, run a task file and (optionally) the stream benchmark, record both.

    python -m hibana_b200.evals.evaluate --target dense-tiny --tasks tasks.jsonl --speed --name trial

The engine is built from the resolved settings (`launch.settings.resolve`, the same resolution `hibana serve`
uses, plus --set KEY=VALUE overrides) and driven through its HTTP app over an in-process ASGI transport, so the
request path (chat template, validation, parsers, detokenisation) is the served one. The task file is JSONL of
{"prompt" | "messages", "answer", "scorer": exact | contains | regex, "max_tokens"}; no dataset ships with this
repository. Output under --out / <name>/: manifest.json (commit, dirty state, settings), served/info.json
(/get_server_info), suite/results.jsonl + summary, speed/ (evals.h2h stream runs), SUMMARY.md. A rerun with the
same name skips finished items. Reference: tools/evaluate.py:1-60.
"""
from __future__ import annotations

import argparse
import asyncio
import hashlib
import json
import subprocess
from pathlib import Path

from .lossy_gate import _parse_sets, score_item


def _git(*args) -> str:
    try:
        return subprocess.run(["git", *args], capture_output=True, text=True, timeout=10).stdout.strip()
    except Exception:  # noqa: BLE001
        return ""


def manifest(cfg) -> dict:
    dirty = _git("status", "--porcelain")
    return {"commit": _git("rev-parse", "HEAD"), "dirty": bool(dirty),
            "dirty_hash": hashlib.sha1(dirty.encode()).hexdigest()[:12] if dirty else "", "config": cfg.as_dict()}


async def run_tasks(client, tasks: list, out_file: Path) -> dict:
    done = {}
    if out_file.exists():
        for line in out_file.read_text().splitlines():
            rec = json.loads(line)
            done[rec["index"]] = rec
    with out_file.open("a") as fh:
        for i, item in enumerate(tasks):
            if i in done:
                continue
            if "messages" in item:
                r = await client.post("/v1/chat/completions", json={"messages": item["messages"],
                                                                    "max_tokens": int(item.get("max_tokens", 128))})
                text = r.json()["choices"][0]["message"]["content"] if r.status_code == 200 else ""
            else:
                r = await client.post("/generate", json={"text": item["prompt"], "sampling_params": {
                    "max_new_tokens": int(item.get("max_tokens", 128))}})
                text = r.json().get("text", "") if r.status_code == 200 else ""
            rec = {"index": i, "status": r.status_code, "output": text, "correct": bool(score_item(text, item))}
            done[i] = rec
            fh.write(json.dumps(rec) + "\n")
            fh.flush()
    n = len(tasks)
    ok = sum(1 for r in done.values() if r["correct"])
    return {"items": n, "correct": ok, "accuracy": ok / max(n, 1)}


async def evaluate(app, cfg, tasks: list, out: Path, speed: bool = False, streams=(1, 4)) -> dict:
    import httpx

    from . import h2h
    out.mkdir(parents=True, exist_ok=True)
    (out / "manifest.json").write_text(json.dumps(manifest(cfg), indent=1))
    summary = {}
    async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://eval", timeout=600) as c:
        (out / "served").mkdir(exist_ok=True)
        (out / "served" / "info.json").write_text(json.dumps((await c.get("/get_server_info")).json(), indent=1,
                                                             default=str))
        if tasks:
            (out / "suite").mkdir(exist_ok=True)
            summary["suite"] = await run_tasks(c, tasks, out / "suite" / "results.jsonl")
        if speed:
            async def post(body):
                return (await c.post("/generate", json=body)).json()
            (out / "speed").mkdir(exist_ok=True)
            runs = [await h2h.run_streams(post, n, duration_s=2.0, warmup_s=0.5, prompt_tokens=32, max_tokens=16)
                    for n in streams]
            (out / "speed" / "streams.json").write_text(json.dumps(runs, indent=1))
            summary["speed"] = runs
    lines = ["# Evaluation summary", ""]
    if "suite" in summary:
        s = summary["suite"]
        lines.append(f"* tasks: {s['correct']} / {s['items']} correct ({100 * s['accuracy']:.1f} %)")
    for r in summary.get("speed", []):
        lines.append(f"* {r['streams']} streams: {r['aggregate_tok_s']:.1f} tok/s aggregate, "
                     f"{r['median_request_tok_s']:.1f} tok/s per request")
    (out / "SUMMARY.md").write_text("\n".join(lines) + "\n")
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--target", default="dense-tiny")
    ap.add_argument("--profile", default="exact")
    ap.add_argument("--set", action="append", default=[])
    ap.add_argument("--tasks", default="")
    ap.add_argument("--speed", action="store_true")
    ap.add_argument("--name", default="run")
    ap.add_argument("--out", default="eval_results")
    args = ap.parse_args(argv)
    from ..api.server import create_app
    from ..engine.llm import LLM
    from ..engine.loop import EngineLoop
    from ..launch.settings import resolve
    from ..tokenizer import load_tokenizer
    cfg = resolve(args.target, profile=args.profile, flags=_parse_sets(args.set))
    llm = LLM(cfg)
    engine = EngineLoop(llm.scheduler).start()
    app = create_app(engine, load_tokenizer(None, llm.target.vocab), model_name=llm.target.name,
                     info={"config": cfg.as_dict()})
    tasks = [json.loads(l) for l in Path(args.tasks).read_text().splitlines() if l.strip()] if args.tasks else []
    summary = asyncio.run(evaluate(app, cfg, tasks, Path(args.out) / args.name, speed=args.speed))
    engine.stop()
    print(json.dumps(summary, indent=1, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
