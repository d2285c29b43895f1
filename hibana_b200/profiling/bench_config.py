"""Full-depth multi-GPU decode benchmark of the hybrid MoE families through the engine.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        -m hibana_b200.profiling.bench_config --family flashnext --mode dpep --batch 256 --prompt 2048

`--mode tp`: tensor parallel over all ranks (mixers by head, shared MLPs by column, experts by range over the
replicated activations, vocabulary-parallel head); every rank holds the whole batch. `--mode dpep`: data-parallel
replicas, each with batch / ranks requests of its own, whose MoE layers share the experts through the all-to-all
over peer memory. The engine is built by `LLM` from an `EngineConfig` (the call a user makes); the model has every
block of the family (no extrapolation), random-init weights of the real geometry, synthetic prompts. One step is
one decode step of the whole (global) batch: device-timed over graph replays and end to end through
`Executor.decode_step` (upload, lockstep round, graph, read-back), max over ranks. Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import time

import torch
import torch.distributed as dist


def main(argv=None, emit=print):
    """Runs the benchmark; rank 0 emits one JSON line and returns the dict (other ranks return None)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="flashnext")
    ap.add_argument("--mode", default="tp", choices=("tp", "dpep"))
    ap.add_argument("--batch", type=int, default=32, help="global batch (dpep: split over the ranks)")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer blocks (marks the result invalid)")
    ap.add_argument("--spec", default="off")
    ap.add_argument("--kv-dtype", default="")
    ap.add_argument("--ssm-state", default="fp32", help="recurrent state format: fp32 | fp16_sr | int8 | int8w")
    args = ap.parse_args(argv)

    from .. import _native as nv
    from ..config import EngineConfig
    from ..engine.llm import LLM
    from ..engine.request import Request, SamplingParams
    from ..target import get_target, scaled

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = control = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    full = get_target(args.family)
    t = scaled(full, layers=args.layers) if args.layers else full
    if args.spec == "off":
        t = scaled(t, mtp_layers=0, mtp_depth=0)
    dp = world if args.mode == "dpep" and world > 1 else 1
    per_rank = args.batch // dp
    assert per_rank >= 1 and per_rank * dp == args.batch, "the global batch must divide over the replicas"
    per_round = 1 if args.spec == "off" else max(t.mtp_depth, 3) + 1      # tokens a round can append
    max_ctx = args.prompt + per_round * (max(args.warmup, 3) + 2 * args.steps) + 64
    cfg = EngineConfig(target=args.family, max_batch=per_rank, max_context=max_ctx, tp=world if dp == 1 else 1, dp=dp,
                       ep=dp if dp > 1 else 1, graph_buckets=f"1,{per_rank}", kv_pages=per_rank * max_ctx + 4096,
                       state_slots=3 * per_rank + 2, spec=args.spec, kv_dtype=args.kv_dtype, ssm_state=args.ssm_state,
                       prefill_budget=max(4096, t.prefill_chunk))
    t0 = time.perf_counter()
    if dp > 1:
        from ..engine.dp import GroupAllGather
        control = GroupAllGather(dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=120)))
        llm = LLM(cfg, target=t, device=dev, control=control, rank=rank)
    else:
        if world > 1:
            from ..parallel.comm import Communicator
            comm = Communicator.create(rank, world, dev, slot_mb=8)
        llm = LLM(cfg, target=t, device=dev, comm=comm)
    build_s = time.perf_counter() - t0
    ex = llm.executor

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        v = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    # tensor-parallel ranks hold the same requests; replicas hold their own
    g = torch.Generator().manual_seed(1234 + (rank if dp > 1 else 0))
    prompts = [torch.randint(0, t.vocab, (args.prompt,), generator=g).tolist() for _ in range(per_rank)]
    reqs = [Request(prompt_ids=p, params=SamplingParams(max_tokens=10 ** 6, ignore_eos=True)) for p in prompts]
    for r in reqs:
        ex.admit(r)
    chunk = min(args.prompt, t.prefill_chunk)
    pre_ms = []
    for r in reqs:
        done = 0
        while done < args.prompt:
            n = min(chunk, args.prompt - done)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ex.prefill_batch([(r, n)])
            e1.record()
            torch.cuda.synchronize()
            pre_ms.append(e0.elapsed_time(e1))
            done += n
    for _ in range(max(args.warmup, 3)):
        ex.decode_step(reqs)
    torch.cuda.synchronize()
    status = nv.read_status(dev)
    if status:
        raise SystemExit(f"device status {status} after warm-up; not timing a failing run")
    steps = args.steps
    sync_all()
    emitted0 = sum(len(r.output_ids) for r in reqs)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        ex.decode_step(reqs)
    e1.record()
    sync_all()
    wall = (time.perf_counter() - w0) * 1e3 / steps
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1) / steps, wall))
    emitted = sum(len(r.output_ids) for r in reqs) - emitted0        # tokens of the timed rounds (this rank)
    per_round_tokens = emitted / max(len(reqs) * steps, 1)
    dev_ms = None
    if args.spec == "off":
        buf = ex.runner.bufs[ex.runner._bucket(per_rank)]
        graph = buf.graph_greedy if getattr(buf, "graph_greedy", None) is not None else buf.graph
        if graph is not None:
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            sync_all()
            dev_ms = max_over_ranks(e0.elapsed_time(e1) / steps)
    status = nv.read_status(dev)
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    if rank == 0:
        pre = sorted(pre_ms)[len(pre_ms) // 2]
        out = {"family": args.family, "mode": args.mode if world > 1 else "single", "n_gpus": world,
               "layers": len(t.layers), "valid": not args.layers, "global_batch": args.batch, "prompt": args.prompt,
               "ms_per_step_e2e": round(e2e_ms, 3),
               "tok_s_e2e": round(args.batch * per_round_tokens / e2e_ms * 1e3, 1),
               "tok_s_per_user_e2e": round(per_round_tokens / e2e_ms * 1e3, 1),
               "prefill_ms_per_chunk": round(pre, 2), "prefill_chunk": chunk, "build_s": round(build_s, 1),
               "launches_per_step": ex.runner.graph_launches.get(per_rank, 0), "device_status": status,
               "peak_alloc_gib": round(mem, 1), "spec": args.spec, "ssm_state": args.ssm_state,
               "data": "synthetic (uniform-random token ids, random-init N(0,0.02) weights)"}
        if dev_ms is not None:
            out.update({"ms_per_step": round(dev_ms, 3), "tok_s": round(args.batch / dev_ms * 1e3, 1),
                        "tok_s_per_user": round(1e3 / dev_ms, 1)})
        if args.spec != "off":
            out["spec_stats"] = ex.spec.stats.as_dict()
            out["tokens_per_round"] = round(per_round_tokens, 3)
            out["rounds_as_graphs"] = ex.spec.graphs.rounds if ex.spec.graphs is not None else 0
        if llm.lockstep is not None:
            out["lockstep_rounds"] = llm.lockstep.rounds
        if emit is not None:
            emit(json.dumps(out))
        return out
    return None
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
