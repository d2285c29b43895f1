"""Cache trace: does a prompt give the same first token and the same last-token activations whichever way its
prefix reached the GPU?

For one prompt the trace runs the engine's own prefill three (optionally four) ways and records, for the last
prompt token, the hidden state entering every block, the final normed state and the first token:
  cold      no cache: the whole prompt is prefilled;
  chunked   no cache, prefilled in small chunks (another kernel shape for the same math);
  cached    the prefix comes from the radix cache (KV slots, and the state snapshot of recurrent layers), only
            the suffix is run;
  restored  (with an SSD tier) the prefix was evicted, came back from disk, then the suffix is run.
`cached` / `restored` against `cold` isolates errors of copies, snapshots and restore (they should be bit-equal for
attention-only models and equal to `chunked` otherwise); `chunked` against `cold` shows what kernel-shape
differences alone do. The report lists, per pair, the first block whose input differs and the largest relative
difference. Recurrent models must run with fp32 states for the comparison to be meaningful.
Reference: hibana/engine/cache_trace.py:30-230.
"""
from __future__ import annotations

import contextlib
import json
from pathlib import Path
from typing import Optional, Sequence

import torch

from .request import Request, SamplingParams


@contextlib.contextmanager
def last_token_trace(model):
    """Records the last row of every sublayer's input while active (wraps each sublayer's `forward`)."""
    stages: dict = {}
    originals = []
    subs = []
    if hasattr(model, "blocks"):
        for bi, blk in enumerate(model.blocks):
            for si, (_, sub) in enumerate(blk.sublayers()):
                if sub is not None:
                    subs.append((f"block{bi}.{'mixer' if si == 0 else 'ffn'}", sub))
    for name, sub in subs:
        orig = sub.forward

        def wrapped(x, *a, _orig=orig, _name=name, **kw):
            stages[_name] = x[-1].detach().float().cpu().clone()
            return _orig(x, *a, **kw)
        sub.forward = wrapped
        originals.append((sub, orig))
    try:
        yield stages
    finally:
        for sub, orig in originals:
            sub.forward = orig


def _prefill(ex, ids: Sequence[int], budget: int) -> tuple:
    """Runs the prompt through admit + chunked prefill; returns (first token, cached prefix length, stages)."""
    r = Request(prompt_ids=list(ids), params=SamplingParams(max_tokens=1))
    with last_token_trace(ex.model) as stages:
        out = ex.generate_batch_requests([r], prefill_budget=budget)[0]
    return out.output_ids[0], stages


def compare(a: dict, b: dict) -> dict:
    first, worst, worst_at = None, 0.0, None
    for name in a:
        if name not in b:
            continue
        d = float((a[name] - b[name]).abs().max() / a[name].abs().max().clamp_min(1e-12))
        if d > 0 and first is None:
            first = name
        if d > worst:
            worst, worst_at = d, name
    return {"first_difference": first, "max_rel_diff": worst, "at": worst_at, "equal": first is None}


def run(make_executor, ids: Sequence[int], prefix_len: int, output: Optional[Path] = None, chunk: int = 16,
        ssd_dir: Optional[str] = None) -> dict:
    """`make_executor()` builds a fresh executor over the same model (fresh pools and cache). `prefix_len` tokens of
    `ids` are first served as their own request so that they sit in the cache for the `cached` run."""
    results, traces = {}, {}
    ex = make_executor()
    results["cold"], traces["cold"] = _prefill(ex, ids, len(ids))
    ex = make_executor()
    results["chunked"], traces["chunked"] = _prefill(ex, ids, chunk)
    ex = make_executor()
    ex.generate_batch_requests([Request(prompt_ids=list(ids[:prefix_len]) + [ids[prefix_len]],
                                        params=SamplingParams(max_tokens=1))])
    hit = ex.state.cache.match(list(ids[:-1]), split=False).length if ex.state.cache is not None else 0
    results["cached"], traces["cached"] = _prefill(ex, ids, len(ids))
    results["cached_prefix"] = hit
    if ssd_dir is not None:
        ex = make_executor()
        ex.enable_ssd_tier(ssd_dir, min_prefix=1, min_gain=1)
        ex.generate_batch_requests([Request(prompt_ids=list(ids[:prefix_len]) + [ids[prefix_len]],
                                            params=SamplingParams(max_tokens=1))])
        ex.persist_prefixes()
        ex.state.cache.flush()
        results["restored"], traces["restored"] = _prefill(ex, ids, len(ids))
        results["restored_tokens"] = ex.stats.get("ssd_restored_tokens", 0)
    report = {"first_tokens": {k: v for k, v in results.items() if isinstance(v, int) and k in traces},
              "cached_prefix": results.get("cached_prefix", 0), "restored_tokens": results.get("restored_tokens"),
              "pairs": {f"{k}_vs_cold": compare(traces["cold"], traces[k]) for k in traces if k != "cold"}}
    if "restored" in traces:
        report["pairs"]["restored_vs_cached"] = compare(traces["cached"], traces["restored"])
    if output is not None:
        output.parent.mkdir(parents=True, exist_ok=True)
        output.write_text(json.dumps(report, indent=1))
        torch.save(traces, output.with_suffix(".pt"))
    return report
