"""Timing hygiene shared by every benchmark: warm-up, L2 flush between iterations, CUDA events on the
launching stream, and roofline fractions against the measured peaks file when present."""
from __future__ import annotations

import json
import statistics
from pathlib import Path
from typing import Callable

import torch

from .. import _native as nv

_FLUSH: dict[int, torch.Tensor] = {}


def flush_l2() -> None:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts from DRAM."""
    dev = torch.cuda.current_device()
    buf = _FLUSH.get(dev)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        _FLUSH[dev] = buf
    buf.zero_()


def time_cuda(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush: bool = True, burst: int = 1) -> dict:
    """Returns {'median_ms', 'min_ms', 'all_ms'} for fn() timed alone on the current stream. `burst` > 1 times that
    many back-to-back calls per sample and reports the mean of each burst: on an idle GPU the first launch of a
    sample starts tens of microseconds after the start event (host launch latency), which a ~100 us kernel would
    otherwise carry in full; only for working sets larger than L2 (nothing is flushed inside a burst)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # a kernel whose bounded wait ran out costs its full limit per launch: never time (or repeat) such a run
    code = nv.read_status()
    if code != 0:
        raise RuntimeError(f"device status {code} after warm-up: a kernel gave up on a wait; not timing it")
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(burst):
            fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / burst)
    return {"median_ms": statistics.median(times), "min_ms": min(times), "all_ms": times}


def measured_peaks() -> dict:
    """Measured per-GPU peaks (copy bandwidth GB/s, bf16 TFLOP/s); falls back to an earlier measurement."""
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
