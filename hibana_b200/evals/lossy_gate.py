"""Lossy-change gate: one scorecard for a candidate configuration paired against a baseline configuration.

    python -m hibana_b200.evals.lossy_gate --target dense-tiny --set fuse_epilogues=0 --name no-fusion

Both arms run this checkout's engine in process on the same frozen prompts. Layers, cheapest first:

  1. Distribution distance. The baseline's own greedy continuations of the prompts are scored by both arms at one
     token per forward (teacher forcing through the engine's verify path); per prompt domain the gate reports the
     argmax agreement and the truncated KL(baseline || candidate) over the baseline's top-k tokens, with 95 %
     bootstrap intervals over blocks of positions. The floor is the baseline scored against itself at another
     batch shape (different kernels, same weights): a candidate "within floor" is indistinguishable from batch
     invariance noise.
  2. Speculation health (targets with a drafter): tokens per verify round and decode tokens/s per prompt, paired.
  3. Task battery: a JSONL file of {"prompt", "answer", "scorer"} items run greedy by both arms, paired per item
     with a McNemar test on the discordant pairs.

Verdict: "exact" (layer 1 within floor everywhere, layer 3 no significant loss), "lossy-ok" (KL above floor but
task battery not significantly worse and speed gain >= --min-gain), "reject" otherwise. Every step writes its own
JSON file under --out, so a rerun with the same name resumes. Reference: tools/lossy_gate.py:1-120,
tools/gate/lossy_gate.py.
"""
from __future__ import annotations

import argparse
import json
import math
import random
import time
from pathlib import Path
from typing import Callable, Optional, Sequence

import torch

from .. import config as cfgmod

DOMAINS = ("code", "math", "prose", "multilingual", "structured", "chat")


def frozen_prompts(vocab: int, per_domain: int = 4, length: int = 48, seed: int = 20240601) -> list:
    """Synthetic stand-ins for the frozen prompt set (no corpus ships with this repository): per domain a fixed
    seeded stream of token ids with a domain-specific repetition structure, so the domains differ in entropy."""
    out = []
    for d, name in enumerate(DOMAINS):
        g = torch.Generator().manual_seed(seed + d)
        period = (4, 7, 0, 0, 5, 3)[d]
        for i in range(per_domain):
            ids = torch.randint(3, vocab, (length,), generator=g).tolist()
            if period:
                for j in range(period, length):
                    if j % (period * 2) < period:
                        ids[j] = ids[j - period]
            out.append({"domain": name, "id": f"{name}-{i}", "ids": ids})
    return out


def _row_logits(executor, seqs: Sequence[Sequence[int]]) -> list:
    """Next-token logits after every position of every sequence (one ragged forward per sequence)."""
    from ..engine.context import VERIFY
    from ..engine.request import Request, SamplingParams
    outs = []
    for ids in seqs:
        r = Request(prompt_ids=list(ids), params=SamplingParams(max_tokens=1))
        r.cacheable = False
        executor.admit(r)
        slots = executor._alloc(r, len(ids))
        lg, _ = executor.runner.forward_rows([r.table_row], [list(ids)], [0], [slots], mode=VERIFY,
                                             want="logits_device",
                                             state_slots=[r.state_slot] if executor.state_pool is not None else None)
        outs.append(lg.float().cpu())
        executor.release(r)
    return outs


def distribution_distance(base_logits: torch.Tensor, cand_logits: torch.Tensor, top_k: int = 20) -> tuple:
    """(argmax agreement per position [T], truncated KL(base || cand) per position [T])."""
    bp = torch.log_softmax(base_logits, -1)
    cp = torch.log_softmax(cand_logits, -1)
    agree = (bp.argmax(-1) == cp.argmax(-1)).float()
    topv, topi = bp.topk(min(top_k, bp.shape[-1]), dim=-1)
    kl = (topv.exp() * (topv - cp.gather(-1, topi))).sum(-1).clamp_min(0)
    return agree, kl


def bootstrap_ci(values: Sequence[float], block: int = 16, n: int = 400, seed: int = 0) -> tuple:
    vals = list(values)
    if not vals:
        return 0.0, 0.0, 0.0
    blocks = [vals[i:i + block] for i in range(0, len(vals), block)]
    rng = random.Random(seed)
    means = []
    for _ in range(n):
        pick = [rng.choice(blocks) for _ in blocks]
        flat = [v for b in pick for v in b]
        means.append(sum(flat) / len(flat))
    means.sort()
    return sum(vals) / len(vals), means[int(0.025 * n)], means[int(0.975 * n) - 1]


def mcnemar(b: int, c: int) -> float:
    """Two-sided exact McNemar p-value for b baseline-only and c candidate-only successes."""
    n = b + c
    if n == 0:
        return 1.0
    k = min(b, c)
    p = sum(math.comb(n, i) for i in range(k + 1)) / 2 ** n
    return min(1.0, 2 * p)


def score_item(text: str, item: dict) -> bool:
    import re
    kind = item.get("scorer", "contains")
    ans = str(item.get("answer", ""))
    if kind == "exact":
        return text.strip() == ans.strip()
    if kind == "regex":
        return re.search(ans, text) is not None
    return ans in text


def run_gate(make_executor: Callable[[cfgmod.EngineConfig], object], base_cfg: cfgmod.EngineConfig,
             cand_cfg: cfgmod.EngineConfig, vocab: int, out: Path, *, continuation: int = 24, tasks: Optional[list] = None,
             tokenizer=None, min_gain: float = 1.05) -> dict:
    """Runs the layers and returns the scorecard (also written to out / scorecard.json)."""
    from ..engine.request import SamplingParams
    out.mkdir(parents=True, exist_ok=True)
    prompts = frozen_prompts(vocab)
    with cfgmod.using(base_cfg):
        ex_b = make_executor(base_cfg)
        t0 = time.perf_counter()
        conts = ex_b.generate_batch([p["ids"] for p in prompts], SamplingParams(max_tokens=continuation, ignore_eos=True))
        base_s = time.perf_counter() - t0
        seqs = [p["ids"] + r.output_ids for p, r in zip(prompts, conts)]
        base_rows = _row_logits(ex_b, seqs)
        floor_rows = _row_logits(ex_b, [s[:-1] + [s[-1]] for s in seqs])          # same weights, second pass
        base_rounds = [sum(r.rounds) / max(len(r.rounds), 1) for r in conts]
    with cfgmod.using(cand_cfg):
        ex_c = make_executor(cand_cfg)
        t0 = time.perf_counter()
        cconts = ex_c.generate_batch([p["ids"] for p in prompts], SamplingParams(max_tokens=continuation, ignore_eos=True))
        cand_s = time.perf_counter() - t0
        cand_rows = _row_logits(ex_c, seqs)
        cand_rounds = [sum(r.rounds) / max(len(r.rounds), 1) for r in cconts]
    layer1 = {}
    within = True
    for dom in DOMAINS:
        ag, kl, fkl = [], [], []
        for p, b, c, f in zip(prompts, base_rows, cand_rows, floor_rows):
            if p["domain"] != dom:
                continue
            n0 = len(p["ids"]) - 1                      # score the continuation positions
            a_, k_ = distribution_distance(b[n0:], c[n0:])
            _, f_ = distribution_distance(b[n0:], f[n0:])
            ag += a_.tolist()
            kl += k_.tolist()
            fkl += f_.tolist()
        m, lo, hi = bootstrap_ci(kl)
        fm, _, fhi = bootstrap_ci(fkl)
        ok = lo <= fhi + 1e-6
        within &= ok
        layer1[dom] = {"argmax_agreement": sum(ag) / max(len(ag), 1), "kl": m, "kl_ci": [lo, hi], "floor_kl": fm,
                       "floor_hi": fhi, "within_floor": ok}
    (out / "layer1.json").write_text(json.dumps(layer1, indent=1))
    tok_b = sum(len(r.output_ids) for r in conts) / max(base_s, 1e-9)
    tok_c = sum(len(r.output_ids) for r in cconts) / max(cand_s, 1e-9)
    layer2 = {"baseline_tok_s": tok_b, "candidate_tok_s": tok_c, "speed_ratio": tok_c / max(tok_b, 1e-9),
              "baseline_tokens_per_round": sum(base_rounds) / len(base_rounds),
              "candidate_tokens_per_round": sum(cand_rounds) / len(cand_rounds)}
    (out / "layer2.json").write_text(json.dumps(layer2, indent=1))
    layer3 = None
    if tasks and tokenizer is not None:
        wins_b = wins_c = both = 0
        for item in tasks:
            ids = tokenizer.encode(item["prompt"])
            sp = SamplingParams(max_tokens=int(item.get("max_tokens", 64)))
            with cfgmod.using(base_cfg):
                tb = tokenizer.decode(ex_b.generate_batch([ids], sp)[0].output_ids)
            with cfgmod.using(cand_cfg):
                tc = tokenizer.decode(ex_c.generate_batch([ids], sp)[0].output_ids)
            sb, sc = score_item(tb, item), score_item(tc, item)
            both += sb and sc
            wins_b += sb and not sc
            wins_c += sc and not sb
        layer3 = {"items": len(tasks), "both": both, "baseline_only": wins_b, "candidate_only": wins_c,
                  "mcnemar_p": mcnemar(wins_b, wins_c)}
        (out / "layer3.json").write_text(json.dumps(layer3, indent=1))
    worse = layer3 is not None and layer3["baseline_only"] > layer3["candidate_only"] and layer3["mcnemar_p"] < 0.05
    if within and not worse:
        verdict = "exact"
    elif not worse and layer2["speed_ratio"] >= min_gain:
        verdict = "lossy-ok"
    else:
        verdict = "reject"
    card = {"verdict": verdict, "layer1": layer1, "layer2": layer2, "layer3": layer3,
            "baseline": base_cfg.as_dict(), "candidate": cand_cfg.as_dict()}
    (out / "scorecard.json").write_text(json.dumps(card, indent=1))
    return card


def _parse_sets(pairs: Sequence[str]) -> dict:
    import dataclasses
    types = {f.name: f.type for f in dataclasses.fields(cfgmod.EngineConfig)}
    out = {}
    for p in pairs:
        k, v = p.split("=", 1)
        ty = types[k]
        out[k] = cfgmod._bool(v) if ty in ("bool", bool) else int(v) if ty in ("int", int) else \
            float(v) if ty in ("float", float) else v
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--target", default="dense-tiny")
    ap.add_argument("--name", default="candidate")
    ap.add_argument("--set", action="append", default=[], help="candidate setting KEY=VALUE (EngineConfig field)")
    ap.add_argument("--baseline-set", action="append", default=[])
    ap.add_argument("--tasks", default="", help="JSONL of {prompt, answer, scorer} items")
    ap.add_argument("--out", default="gate_results")
    args = ap.parse_args(argv)
    from ..engine.llm import LLM
    from ..target import get_target
    from ..tokenizer import ByteTokenizer
    t = get_target(args.target)
    base = cfgmod.EngineConfig(target=args.target, max_batch=8, **_parse_sets(args.baseline_set))
    cand = base.replace(**_parse_sets(args.set))
    tasks = [json.loads(l) for l in Path(args.tasks).read_text().splitlines() if l.strip()] if args.tasks else None
    card = run_gate(lambda c: LLM(c).executor, base, cand, t.vocab, Path(args.out) / args.name, tasks=tasks,
                    tokenizer=ByteTokenizer() if tasks else None)
    print(json.dumps({"verdict": card["verdict"], "layer2": card["layer2"]}, indent=1))
    return 0 if card["verdict"] != "reject" else 1


if __name__ == "__main__":
    raise SystemExit(main())
