"""Timing hygiene shared by every benchmark: warm-up, L2 flush between iterations, CUDA events on the
launching stream, and roofline fractions against the measured peaks file when present."""
from __future__ import annotations

import json
import statistics
from pathlib import Path
from typing import Callable

import torch

_FLUSH: dict[int, torch.Tensor] = {}


def flush_l2() -> None:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts from DRAM."""
    dev = torch.cuda.current_device()
    buf = _FLUSH.get(dev)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        _FLUSH[dev] = buf
    buf.zero_()


def time_cuda(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush: bool = True) -> dict:
    """Returns {'median_ms', 'min_ms', 'all_ms'} for fn() timed alone on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    return {"median_ms": statistics.median(times), "min_ms": min(times), "all_ms": times}


def measured_peaks() -> dict:
    """Measured per-GPU peaks (copy bandwidth GB/s, bf16 TFLOP/s); falls back to an earlier measurement."""
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
