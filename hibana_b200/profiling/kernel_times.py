"""Per-kernel device time of a few decode steps of a hybrid family (or the dense decoder), from CUPTI through
torch.profiler.

    python -m hibana_b200.profiling.kernel_times --family nemotron --layers 18 --batch 16 --prompt 512

Builds the first `--layers` blocks at full width with random-init weights, prefills `--batch` synthetic prompts, runs
three eager decode steps to warm up and profiles `--steps` more. Prints the kernels by total device time with their
call counts. The times are taken under a profiler: use them to compare SHARES and to find outliers, never as
benchmark values (bench_family / bench_config time the same steps with CUDA events).
"""
from __future__ import annotations

import argparse

import torch
from torch.profiler import ProfilerActivity, profile

from ..engine.executor import Executor
from ..engine.request import Request, SamplingParams
from ..target import get_target, scaled


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="nemotron")
    ap.add_argument("--layers", type=int, default=18)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--prefill", action="store_true",
                    help="profile the prefill of one fresh request of --prompt tokens instead of decode steps")
    args = ap.parse_args()
    t = scaled(get_target(args.family), layers=args.layers, mtp_layers=0)
    dev = torch.device("cuda")
    if t.family == "dense":
        from ..models.dense import DenseModel
        model = DenseModel(t, dev, seed=0)
    else:
        from ..models.hybrid import HybridModel
        model = HybridModel(t, dev, seed=0)
    ex = Executor(model, max_batch=args.batch, max_ctx=args.prompt + 64, use_graphs=False, radix_cache=not args.prefill)
    g = torch.Generator().manual_seed(1)
    if args.prefill:
        def one_prefill(seed):
            gg = torch.Generator().manual_seed(seed)
            r = Request(prompt_ids=torch.randint(0, t.vocab, (args.prompt,), generator=gg).tolist(),
                        params=SamplingParams(max_tokens=1, ignore_eos=True))
            ex.admit(r)
            done = 0
            while done < args.prompt:
                n = min(t.prefill_chunk, args.prompt - done)
                ex.prefill_batch([(r, n)])
                done += n
            ex.release(r)
        for s_ in range(3):
            one_prefill(s_)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            one_prefill(9)
            torch.cuda.synchronize()
        rows = sorted((e for e in prof.key_averages() if e.self_device_time_total > 0),
                      key=lambda e: -e.self_device_time_total)
        total = sum(e.self_device_time_total for e in rows)
        print(f"{args.family}: {args.layers} blocks, prefill of {args.prompt} tokens, {total / 1e3:.3f} ms of kernels")
        for e in rows[:args.rows]:
            print(f"{e.self_device_time_total:9.1f} us {e.count:5d} calls "
                  f"{e.self_device_time_total / max(e.count, 1):8.1f} us/call  {e.key[:110]}")
        return
    prompts = [torch.randint(0, t.vocab, (args.prompt,), generator=g).tolist() for _ in range(args.batch)]
    reqs = [Request(prompt_ids=p, params=SamplingParams(max_tokens=10 ** 6, ignore_eos=True)) for p in prompts]
    for i in range(0, args.batch, 4):
        for r in reqs[i:i + 4]:
            ex.admit(r)
        ex.prefill_batch([(r, args.prompt) for r in reqs[i:i + 4]])
    for _ in range(3):
        ex.decode_step(reqs)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            ex.decode_step(reqs)
        torch.cuda.synchronize()
    rows = sorted((e for e in prof.key_averages() if e.self_device_time_total > 0),
                  key=lambda e: -e.self_device_time_total)
    total = sum(e.self_device_time_total for e in rows)
    print(f"{args.family}: {args.layers} blocks, batch {args.batch}, {args.steps} decode steps, "
          f"{total / 1e3 / args.steps:.3f} ms of kernels per step")
    for e in rows[:args.rows]:
        print(f"{e.self_device_time_total / args.steps:9.1f} us/step {e.count // args.steps:5d} calls/step "
              f"{e.self_device_time_total / max(e.count, 1):8.1f} us/call  {e.key[:110]}")


if __name__ == "__main__":
    main()
