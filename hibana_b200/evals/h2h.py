"""Head-to-head speed of two served builds, as a client sees them.

    python -m hibana_b200.evals.h2h --base http://127.0.0.1:30001 --cand http://127.0.0.1:30002 --streams 1,8,32

Per arm and stream count N: N closed-loop streams each send their next `/generate` request as soon as the previous
one ends (numbered prompts, so no two share a prefix), tokens are counted over --duration-s after --warmup-s, and
the table reports aggregate output tokens/s, the median per-request decode tokens/s and the median time to first
token. Arms are alternated `--repeats` times and averaged. The result is one Markdown table (and results.json) to
paste into a change description. Reference: tools/h2h_pr.py:1-60 (what is measured and how the arms alternate).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import statistics
import time
from pathlib import Path
from typing import Callable, Optional


async def _stream(post: Callable, stream_id: int, prompt_tokens: int, max_tokens: int, stop_at: float,
                  count_from: float, records: list) -> None:
    n = 0
    while time.monotonic() < stop_at:
        n += 1
        ids = [(stream_id * 7919 + n * 104729 + j * 31) % 2000 + 3 for j in range(prompt_tokens)]
        t0 = time.monotonic()
        out = await post({"input_ids": ids, "sampling_params": {"max_new_tokens": max_tokens, "ignore_eos": True}})
        t1 = time.monotonic()
        if t0 >= count_from:
            meta = out.get("meta_info", {})
            records.append({"tokens": int(meta.get("completion_tokens", 0)), "seconds": t1 - t0,
                            "ttft": meta.get("ttft_s")})


async def run_streams(post: Callable, streams: int, *, duration_s: float = 10.0, warmup_s: float = 2.0,
                      prompt_tokens: int = 256, max_tokens: int = 128) -> dict:
    """`post(body) -> awaitable dict` sends one /generate request."""
    start = time.monotonic()
    records: list = []
    await asyncio.gather(*[_stream(post, i, prompt_tokens, max_tokens, start + warmup_s + duration_s,
                                   start + warmup_s, records) for i in range(streams)])
    total = sum(r["tokens"] for r in records)
    span = max(time.monotonic() - start - warmup_s, 1e-9)
    per_req = [r["tokens"] / r["seconds"] for r in records if r["seconds"] > 0 and r["tokens"]]
    ttfts = [r["ttft"] for r in records if r.get("ttft") is not None]
    return {"streams": streams, "requests": len(records), "aggregate_tok_s": total / span,
            "median_request_tok_s": statistics.median(per_req) if per_req else 0.0,
            "median_ttft_s": statistics.median(ttfts) if ttfts else None}


def http_poster(url: str):
    import httpx
    client = httpx.AsyncClient(base_url=url, timeout=600)

    async def post(body: dict) -> dict:
        r = await client.post("/generate", json=body)
        r.raise_for_status()
        return r.json()
    return post


def markdown(results: dict) -> str:
    lines = ["| streams | base tok/s | cand tok/s | ratio | base req tok/s | cand req tok/s |", "|---|---|---|---|---|---|"]
    for n in sorted(results["base"]):
        b, c = results["base"][n], results["cand"][n]
        lines.append(f"| {n} | {b['aggregate_tok_s']:.1f} | {c['aggregate_tok_s']:.1f} | "
                     f"{c['aggregate_tok_s'] / max(b['aggregate_tok_s'], 1e-9):.3f} | "
                     f"{b['median_request_tok_s']:.1f} | {c['median_request_tok_s']:.1f} |")
    return "\n".join(lines)


async def head_to_head(base_post: Callable, cand_post: Callable, stream_counts, repeats: int = 1, **kw) -> dict:
    acc: dict = {"base": {}, "cand": {}}
    for _ in range(repeats):
        for arm, post in (("base", base_post), ("cand", cand_post)):      # alternated: drift hits both arms alike
            for n in stream_counts:
                acc[arm].setdefault(n, []).append(await run_streams(post, n, **kw))
    out: dict = {"base": {}, "cand": {}}
    for arm in acc:
        for n, runs in acc[arm].items():
            out[arm][n] = {k: (statistics.mean(r[k] for r in runs) if isinstance(runs[0][k], (int, float)) else runs[0][k])
                           for k in runs[0]}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--base", required=True)
    ap.add_argument("--cand", required=True)
    ap.add_argument("--streams", default="1,8,32")
    ap.add_argument("--repeats", type=int, default=1)
    ap.add_argument("--duration-s", type=float, default=10.0)
    ap.add_argument("--warmup-s", type=float, default=2.0)
    ap.add_argument("--out", default="h2h_results")
    args = ap.parse_args(argv)
    counts = [int(x) for x in args.streams.split(",")]
    res = asyncio.run(head_to_head(http_poster(args.base), http_poster(args.cand), counts, args.repeats,
                                   duration_s=args.duration_s, warmup_s=args.warmup_s))
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    (out / "results.json").write_text(json.dumps(res, indent=1))
    table = markdown(res)
    (out / "report.md").write_text(table + "\n")
    print(table)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
