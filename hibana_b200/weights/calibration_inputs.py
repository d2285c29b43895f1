"""Calibration samples for the 3-bit copies: prompts answered by the target itself, rendered with its chat template.

Three steps, each a sub-command; every capture (`weights/calibrate_model.py --inputs`) reads the last one's file.

1. `prompts`: first user turns from local prompt files (one "source" per file: .jsonl / .json records with
   `messages`, `conversations`, `prompt`, `question` or `text`; .txt with one prompt per blank-line-separated
   paragraph; .parquet when pyarrow is there), an equal seeded draw from each source, so that one large source does
   not decide what the routed experts see. A prompt that shares a 13-word span with an evaluation set (`--evals`: a
   directory of .jsonl / .tsv question files), or equals a shorter evaluation question, is dropped; labels and
   reference answers are never read. Nothing is downloaded: the files are whatever the operator has on disk.
2. `generate --url`: the served target answers each prompt (its own distribution: serve it without the 3-bit copies
   being fitted). Answers append to OUTPUT.partial.jsonl as they finish, so an interrupted run resumes.
3. `build --target`: each answered turn rendered with the target's chat template (its reasoning in `<think>`, then
   the answer) and tokenised with its tokenizer; a turn longer than `--max-tokens` is cut, shorter ones are packed
   whole into samples of up to `--max-tokens` tokens.

    python -m hibana_b200.weights.calibration_inputs prompts --sources chat.jsonl code.jsonl --evals evals/ --output prompts.json
    python -m hibana_b200 serve qwen38 --profile exact &
    python -m hibana_b200.weights.calibration_inputs generate --prompts prompts.json --url http://127.0.0.1:30001 --output answers.json
    python -m hibana_b200.weights.calibration_inputs build --target qwen38 --answers answers.json --weights CKPT --output samples.json

Reference: hibana/weights/calibration_inputs.py:1-24 (the same three steps over downloaded datasets).
"""
from __future__ import annotations

import argparse
import csv
import hashlib
import json
import random
import re
import threading
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Callable, Iterable, Optional, Sequence

SPAN = 13                      # words in a shared span that marks a prompt as an evaluation item
VERSION = "hibana_b200-calibration-inputs-v1"
PROMPT_FIELDS = ("prompt", "question", "problem", "text", "source", "Question", "instruction")
_WORD = re.compile(r"[0-9a-z]+")


# ---- text helpers
def words(text: str) -> list[str]:
    return _WORD.findall(text.lower())


def span_hashes(text: str, n: int = SPAN) -> set:
    w = words(text)
    return {hash(" ".join(w[i:i + n])) for i in range(len(w) - n + 1)}


def first_user_turn(record) -> Optional[str]:
    """The first user message of a record in any of the common shapes (None when it has none)."""
    if isinstance(record, str):
        return record.strip() or None
    if not isinstance(record, dict):
        return None
    for key in ("messages", "conversations", "conversation"):
        turns = record.get(key)
        if isinstance(turns, list):
            for t in turns:
                if not isinstance(t, dict):
                    continue
                role = t.get("role", t.get("from", ""))
                if role in ("user", "human"):
                    text = t.get("content", t.get("value", ""))
                    return text.strip() if isinstance(text, str) and text.strip() else None
            return None
    for key in PROMPT_FIELDS:
        v = record.get(key)
        if isinstance(v, str) and v.strip():
            return v.strip()
    return None


def read_records(path) -> list:
    p = Path(path)
    suffix = p.suffix.lower()
    if suffix == ".jsonl":
        return [json.loads(line) for line in p.read_text().splitlines() if line.strip()]
    if suffix == ".json":
        data = json.loads(p.read_text())
        return data if isinstance(data, list) else data.get("prompts", data.get("data", []))
    if suffix == ".tsv":
        with open(p, newline="") as f:
            return [row[0] for row in csv.reader(f, delimiter="\t") if row]
    if suffix == ".parquet":
        try:
            import pyarrow.parquet as pq
        except ImportError as exc:
            raise ImportError(f"{p}: parquet prompt files need pyarrow") from exc
        return pq.read_table(str(p)).to_pylist()
    return [para for para in re.split(r"\n\s*\n", p.read_text()) if para.strip()]


def load_prompts(path) -> list[str]:
    out = []
    for rec in read_records(path):
        text = first_user_turn(rec)
        if text:
            out.append(text)
    return out


# ---- step 1: prompts
class EvalFilter:
    """Drops prompts that are evaluation items: a shared 13-word span, or equality with a shorter question."""

    def __init__(self, questions: Iterable[str] = ()):
        self.spans: set = set()
        self.short: set = set()
        for q in questions:
            w = words(q)
            if len(w) >= SPAN:
                self.spans |= span_hashes(q)
            elif w:
                self.short.add(" ".join(w))

    @classmethod
    def from_directory(cls, directory) -> "EvalFilter":
        qs = []
        for p in sorted(Path(directory).rglob("*")):
            if p.suffix.lower() in (".jsonl", ".json", ".tsv", ".txt"):
                qs += load_prompts(p)
        return cls(qs)

    def __call__(self, prompt: str) -> bool:
        w = words(prompt)
        if " ".join(w) in self.short:
            return True
        return bool(self.spans) and not self.spans.isdisjoint(span_hashes(prompt))


def draw(by_source: dict, per_source: int, seed: int = 0, is_eval: Optional[Callable[[str], bool]] = None) -> list[dict]:
    """An equal seeded draw from every source, evaluation items and duplicates dropped first."""
    out, seen = [], set()
    for source in sorted(by_source):
        pool = []
        for text in by_source[source]:
            key = hashlib.blake2b(" ".join(words(text)).encode(), digest_size=12).digest()
            if key in seen or (is_eval is not None and is_eval(text)):
                continue
            seen.add(key)
            pool.append(text)
        rng = random.Random(f"{seed}:{source}")
        rng.shuffle(pool)
        out += [{"source": source, "prompt": t} for t in pool[:per_source]]
    return out


def cmd_prompts(args) -> dict:
    is_eval = EvalFilter.from_directory(args.evals) if args.evals else None
    by_source = {Path(p).stem: load_prompts(p) for p in args.sources}
    picked = draw(by_source, args.per_source, args.seed, is_eval)
    doc = {"version": VERSION, "seed": args.seed, "per_source": args.per_source,
           "sources": {s: len(v) for s, v in by_source.items()}, "prompts": picked}
    Path(args.output).write_text(json.dumps(doc, indent=1))
    return {"prompts": len(picked), "sources": len(by_source), "output": args.output}


# ---- step 2: generate
def ask_server(url: str, prompt: str, max_tokens: int, temperature: float, timeout: float = 1800.0) -> dict:
    body = json.dumps({"messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens,
                       "temperature": temperature}).encode()
    req = urllib.request.Request(url.rstrip("/") + "/v1/chat/completions", data=body,
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        msg = json.loads(r.read())["choices"][0]["message"]
    return {"reasoning": msg.get("reasoning_content") or "", "answer": msg.get("content") or ""}


def generate(prompts: Sequence[dict], output, ask: Callable[[str], dict], concurrency: int = 8) -> list[dict]:
    """Answers every prompt through `ask`; finished answers are appended to OUTPUT.partial.jsonl at once and a rerun
    skips them. Returns (and writes) the answers in the prompts' order."""
    out = Path(output)
    partial = out.with_suffix(out.suffix + ".partial.jsonl")
    done: dict = {}
    if partial.exists():
        for line in partial.read_text().splitlines():
            if line.strip():
                rec = json.loads(line)
                done[rec["prompt"]] = rec
    lock = threading.Lock()

    def one(item):
        if item["prompt"] in done:
            return
        rec = dict(item, **ask(item["prompt"]))
        with lock:
            done[item["prompt"]] = rec
            with open(partial, "a") as f:
                f.write(json.dumps(rec) + "\n")
    with ThreadPoolExecutor(max_workers=max(1, concurrency)) as pool:
        list(pool.map(one, prompts))
    answers = [done[p["prompt"]] for p in prompts if p["prompt"] in done]
    out.write_text(json.dumps({"version": VERSION, "answers": answers}, indent=1))
    return answers


def cmd_generate(args) -> dict:
    prompts = json.loads(Path(args.prompts).read_text())["prompts"]
    answers = generate(prompts, args.output,
                       lambda p: ask_server(args.url, p, args.max_tokens, args.temperature), args.concurrency)
    return {"answers": len(answers), "output": args.output}


# ---- step 3: build
def render_turn(template, prompt: str, reasoning: str, answer: str) -> str:
    """The conversation as the target saw and wrote it: its reasoning in <think>, then the answer."""
    reply = (f"<think>\n{reasoning.strip()}\n</think>\n\n" if reasoning.strip() else "") + answer.strip()
    return template.render([{"role": "user", "content": prompt}, {"role": "assistant", "content": reply}],
                           add_generation_prompt=False)


def pack(turns: Sequence[Sequence[int]], max_tokens: int) -> list[list[int]]:
    """A turn longer than `max_tokens` is cut; shorter ones go whole into samples of up to `max_tokens` tokens, in
    order (a sample is closed when the next turn does not fit)."""
    samples, cur = [], []
    for ids in turns:
        ids = list(ids)[:max_tokens]
        if not ids:
            continue
        if len(cur) + len(ids) > max_tokens:
            samples.append(cur)
            cur = []
        cur = cur + ids
    if cur:
        samples.append(cur)
    return samples


def build(answers: Sequence[dict], template, tokenizer, max_tokens: int = 2048) -> list[list[int]]:
    turns = [tokenizer.encode(render_turn(template, a["prompt"], a.get("reasoning", ""), a.get("answer", "")))
             for a in answers if a.get("answer") or a.get("reasoning")]
    return pack(turns, max_tokens)


def cmd_build(args) -> dict:
    from ..api.chat_template import ChatTemplate
    from ..target import get_target
    from ..tokenizer import load_tokenizer
    t = get_target(args.target)
    answers = json.loads(Path(args.answers).read_text())["answers"]
    samples = build(answers, ChatTemplate.load(args.weights or None), load_tokenizer(args.weights or None, t.vocab),
                    args.max_tokens)
    Path(args.output).write_text(json.dumps({"version": VERSION, "target": t.name, "max_tokens": args.max_tokens,
                                             "samples": samples}))
    return {"samples": len(samples), "tokens": sum(len(s) for s in samples), "output": args.output}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prompts")
    p.add_argument("--sources", nargs="+", required=True, help="prompt files, one source each")
    p.add_argument("--evals", default="", help="directory of evaluation question files to keep out of the draw")
    p.add_argument("--per-source", type=int, default=512)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--output", required=True)
    p.set_defaults(run=cmd_prompts)
    p = sub.add_parser("generate")
    p.add_argument("--prompts", required=True)
    p.add_argument("--url", required=True)
    p.add_argument("--max-tokens", type=int, default=4096)
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--concurrency", type=int, default=8)
    p.add_argument("--output", required=True)
    p.set_defaults(run=cmd_generate)
    p = sub.add_parser("build")
    p.add_argument("--target", required=True)
    p.add_argument("--answers", required=True)
    p.add_argument("--weights", default="", help="checkpoint directory (tokenizer and chat template); default: the "
                                                  "byte tokenizer and the built-in template")
    p.add_argument("--max-tokens", type=int, default=2048)
    p.add_argument("--output", required=True)
    p.set_defaults(run=cmd_build)
    args = ap.parse_args(argv)
    print(json.dumps(args.run(args)))


if __name__ == "__main__":
    main()
