"""Per-layer timing of the hybrid model families at their real dimensions on one GPU.

    python -m hibana_b200.profiling.bench_family --family flashnext --layers 8 --batch 32 --prompt 4096

Builds the first `--layers` blocks of the family (random-init weights of the real geometry, NVFP4 where the
family uses it), prefills `--batch` synthetic prompts, then times decode steps with CUDA events (graph replay) and
one prefill chunk. Prints per-block milliseconds and the figure extrapolated to the family's full depth (blocks are
periodic, so `layers` should be a multiple of the pattern period: 4 for flashnext / qwen38, 9-10 for nemotron).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..engine.executor import Executor
from ..engine.request import Request, SamplingParams
from ..models.hybrid import HybridModel
from ..target import get_target, scaled


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="flashnext")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--kv-dtype", default="bf16")
    args = ap.parse_args()
    full = get_target(args.family)
    t = scaled(full, layers=args.layers, kv_dtype=args.kv_dtype, mtp_layers=0)
    dev = torch.device("cuda")
    model = HybridModel(t, dev, seed=0)
    batch, plen = args.batch, args.prompt
    max_ctx = plen + args.steps + 16
    ex = Executor(model, max_batch=batch, max_ctx=max_ctx, kv_slots=batch * max_ctx + 1024, use_graphs=True,
                  buckets=(batch,))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, t.vocab, (plen,), generator=g).tolist() for _ in range(batch)]

    def calib():
        r = Request(prompt_ids=prompts[0][:256], params=SamplingParams(max_tokens=1))
        ex.admit(r)
        ex.prefill_batch([(r, 256)])
        ex.release(r)
    model.calibrate(calib)
    reqs = [Request(prompt_ids=p, params=SamplingParams(max_tokens=10_000, ignore_eos=True)) for p in prompts]
    chunk = min(plen, t.prefill_chunk)
    pre_ms = []
    for r in reqs:
        ex.admit(r)
        done = 0
        while done < plen:
            n = min(chunk, plen - done)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ex.prefill_batch([(r, n)])
            e1.record()
            torch.cuda.synchronize()
            pre_ms.append(e0.elapsed_time(e1) / n * chunk)
            done += n
    ex.capture_graphs()
    for _ in range(3):
        ex.decode_step(reqs)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ex.decode_step(reqs)
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / args.steps
    depth = len(full.layers)
    scale = depth / args.layers
    # the output head (lm_head GEMM + argmax) runs once per step whatever the depth: time it alone and keep it out
    # of the per-block figure
    from ..ops import sampling
    from .timing import time_cuda
    hx = torch.randn(batch, t.hidden, device=dev).to(torch.bfloat16)
    head_ms = time_cuda(lambda: sampling.argmax(model.logits(hx)), iters=10)["median_ms"]
    head_ms = min(head_ms, 0.9 * step_ms)
    block_ms = (step_ms - head_ms) / args.layers
    full_step_ms = block_ms * depth + head_ms
    pre = sorted(pre_ms)[len(pre_ms) // 2]
    from .. import _native as nv
    print(json.dumps({
        "family": args.family, "layers_built": args.layers, "layers_full": depth, "batch": batch, "prompt": plen,
        "decode_ms_per_step": round(step_ms, 3), "head_ms": round(head_ms, 3),
        "decode_ms_per_block": round(block_ms, 4),
        "decode_tok_s_at_full_depth": round(batch / full_step_ms * 1e3, 1),
        "prefill_ms_per_chunk": round(pre, 2), "prefill_chunk": chunk,
        "prefill_tok_s_at_full_depth": round(chunk / (pre * scale) * 1e3, 1),
        "note": "decode: (step - output head) / built blocks x full depth + output head; prefill: linear in depth",
        "device_status": nv.read_status(dev)}))


if __name__ == "__main__":
    main()
