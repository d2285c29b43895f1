"""Agent-session prefix-cache workload: concurrent sessions that share one long prefix and grow turn by turn.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        -m hibana_b200.profiling.agent_sessions --sessions 64 --prefix 32768 --turns 8 --append 2048 --gen 256 --w3

Every session's prompt is the shared prefix, then per turn `--append` fresh random tokens followed by `--gen`
generated ones; a turn's prompt is the session's whole conversation so far, so the radix cache serves the shared
prefix to every session and each session's own history to its next turn. `--kv-slots` caps the KV pool so that
sessions evict one another between turns; with `--ssd-dir` evicted prefixes are backed up to disk and restored at the
next turn instead of being prefilled again. The engine is built once by `LLM` (3-bit decode copies with `--w3`,
CUDA-graph decode) and serves the turns through its scheduler; reported per turn: p50 / max time to first token over
the sessions, cached and restored tokens, and the decode rate. One JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import time

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--target", default="dense-27b")
    ap.add_argument("--sessions", type=int, default=64)
    ap.add_argument("--prefix", type=int, default=32768)
    ap.add_argument("--turns", type=int, default=8)
    ap.add_argument("--append", type=int, default=2048)
    ap.add_argument("--gen", type=int, default=256)
    ap.add_argument("--w3", action="store_true")
    ap.add_argument("--ssd-dir", default="")
    ap.add_argument("--kv-slots", type=int, default=0, help="cap of the KV pool in tokens (0: everything fits)")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (marks the result invalid)")
    ap.add_argument("--kv-dtype", default="")
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args()

    from .. import _native as nv
    from ..config import EngineConfig
    from ..engine.llm import LLM
    from ..engine.request import SamplingParams
    from ..target import get_target, scaled

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = args.device == "cuda"
    dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    comm = None
    if on_gpu:
        torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.comm import Communicator
        comm = Communicator.create(rank, world, dev, slot_mb=8)
    t = get_target(args.target)
    if args.layers:
        t = scaled(t, layers=args.layers)
    conv = args.prefix + args.turns * (args.append + args.gen)
    need = args.prefix + args.sessions * (conv - args.prefix) + 8192
    slots = min(need, args.kv_slots) if args.kv_slots else need
    cfg = EngineConfig(target=args.target, max_batch=args.sessions, max_context=conv + 64, tp=world, w3=args.w3,
                       kv_pages=slots, ssd_dir=args.ssd_dir, ssd_min_prefix=1024, ssd_min_gain=512,
                       kv_dtype=args.kv_dtype, cuda_graphs=on_gpu, graph_buckets=f"1,8,{args.sessions}",
                       prefill_budget=8192, prefill_chunk=2048)
    t0 = time.perf_counter()
    llm = LLM(cfg, target=t, device=dev, comm=comm)
    build_s = time.perf_counter() - t0
    ex = llm.executor
    g = torch.Generator().manual_seed(77)                      # the same workload on every rank
    prefix = torch.randint(0, t.vocab, (args.prefix,), generator=g).tolist()
    history = [list(prefix) for _ in range(args.sessions)]
    sp = SamplingParams(max_tokens=args.gen, ignore_eos=True)
    # the shared prefix is a system prompt: it is in the cache before the sessions start (timed separately)
    w0 = time.perf_counter()
    llm.generate([list(prefix) + [1]], SamplingParams(max_tokens=1, ignore_eos=True))
    if on_gpu:
        torch.cuda.synchronize()
    prefix_s = time.perf_counter() - w0
    turns = []
    for turn in range(args.turns):
        for h in history:
            h.extend(torch.randint(0, t.vocab, (args.append,), generator=g).tolist())
        cached0 = ex.stats.get("cached_tokens", 0)
        restored0 = ex.ssd.restored_tokens if ex.ssd is not None else 0
        pre0 = ex.stats.get("prefill_tokens", 0)
        w0 = time.perf_counter()
        reqs = llm.generate([list(h) for h in history], sp)
        if on_gpu:
            torch.cuda.synchronize()
        wall = time.perf_counter() - w0
        for h, r in zip(history, reqs):
            h.extend(r.output_ids)
        ttft = sorted(r.ttft for r in reqs if r.ttft is not None)
        turns.append({"turn": turn + 1, "ttft_p50_s": round(statistics.median(ttft), 3) if ttft else None,
                      "ttft_max_s": round(ttft[-1], 3) if ttft else None, "wall_s": round(wall, 2),
                      "cached_tokens": ex.stats.get("cached_tokens", 0) - cached0,
                      "restored_tokens": (ex.ssd.restored_tokens - restored0) if ex.ssd is not None else 0,
                      "prefilled_tokens": ex.stats.get("prefill_tokens", 0) - pre0,
                      "generated": sum(len(r.output_ids) for r in reqs)})
    status = nv.read_status(dev) if on_gpu else 0
    if rank == 0:
        gen = sum(x["generated"] for x in turns)
        print(json.dumps({"workload": "agent sessions", "target": t.name, "layers": len(t.layers),
                          "valid": not args.layers, "n_gpus": world, "sessions": args.sessions, "prefix": args.prefix,
                          "turns": args.turns, "append": args.append, "gen": args.gen, "w3": args.w3,
                          "ssd_tier": bool(args.ssd_dir), "kv_slots": slots, "kv_slots_needed": need,
                          "build_s": round(build_s, 1), "prefix_prefill_s": round(prefix_s, 2), "total_wall_s": round(sum(x["wall_s"] for x in turns), 1),
                          "generated_tok_s_overall": round(gen / max(sum(x["wall_s"] for x in turns), 1e-9), 1),
                          "per_turn": turns, "ssd": ex.ssd.stats() if ex.ssd is not None else None,
                          "device_status": status,
                          "data": "synthetic (uniform-random token ids, random-init weights)"}), flush=True)
    llm.shutdown()
    if world > 1:
        dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
