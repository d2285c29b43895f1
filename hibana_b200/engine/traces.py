"""Request traces: one JSON line per finished request, written by a background thread through a bounded queue,
rotated at 64 MiB, oldest files pruned above the cap. Reference: hibana/engine/traces.py:1-227 (FORMAT_VERSION 4)."""
from __future__ import annotations

import json
import queue
import threading
import time
from pathlib import Path

FORMAT_VERSION = 4
ROTATE_BYTES = 64 << 20


class TraceSink:
    def __init__(self, directory: str, cap_bytes: int = 32 << 30, depth: int = 4096):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.cap = cap_bytes
        self.q: "queue.Queue" = queue.Queue(maxsize=depth)
        self.dropped = 0
        self._file = None
        self._size = 0
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._run, name="hibana-traces", daemon=True)
        self.thread.start()

    def record(self, req) -> None:
        rec = {"v": FORMAT_VERSION, "t": time.time(), "rid": req.rid, "prompt_ids": req.prompt_ids,
               "output_ids": req.output_ids, "finish": req.finish_reason, "cached": req.cached_len,
               "ttft": req.ttft, "rounds": req.rounds,
               "params": {"temperature": req.params.temperature, "top_k": req.params.top_k, "top_p": req.params.top_p,
                          "max_tokens": req.params.max_tokens}}
        try:
            self.q.put_nowait(rec)
        except queue.Full:
            self.dropped += 1

    def _open(self) -> None:
        if self._file is not None:
            self._file.close()
        self._file = open(self.dir / f"traces-{int(time.time() * 1e3)}.jsonl", "a")
        self._size = 0
        files = sorted(self.dir.glob("traces-*.jsonl"))
        total = sum(f.stat().st_size for f in files)
        while total > self.cap and len(files) > 1:
            total -= files[0].stat().st_size
            files.pop(0).unlink()

    def _run(self) -> None:
        while not self._stop.is_set() or not self.q.empty():
            try:
                rec = self.q.get(timeout=0.2)
            except queue.Empty:
                continue
            if self._file is None or self._size > ROTATE_BYTES:
                self._open()
            line = json.dumps(rec) + "\n"
            self._file.write(line)
            self._file.flush()
            self._size += len(line)

    def close(self) -> None:
        self._stop.set()
        self.thread.join(5)
        if self._file is not None:
            self._file.close()


def summarize(directory: str) -> dict:
    n = out_tokens = cached = 0
    rounds = []
    ttfts = []
    for f in sorted(Path(directory).glob("traces-*.jsonl")):
        for line in f.read_text().splitlines():
            try:
                r = json.loads(line)
            except json.JSONDecodeError:
                continue
            n += 1
            out_tokens += len(r.get("output_ids", []))
            cached += r.get("cached", 0)
            rounds.extend(r.get("rounds") or [])
            if r.get("ttft") is not None:
                ttfts.append(r["ttft"])
    ttfts.sort()
    return {"requests": n, "output_tokens": out_tokens, "cached_tokens": cached,
            "tokens_per_round": (sum(rounds) / len(rounds)) if rounds else None,
            "ttft_p50": ttfts[len(ttfts) // 2] if ttfts else None}
