"""Headline benchmark: decode throughput of the 27B-class dense NVFP4 decoder (batch 64, 2048-token prompts).

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torch.distributed.run)

One "step" is one decode step of the whole batch. `value` is the aggregate output tokens/s over all GPUs, timed
on the device with CUDA events around K graph replays of the full step (embedding -> 64 layers -> lm_head ->
sampling), max over ranks. `e2e` is the same metric through the public engine API (`Executor.decode_step`),
including each step's pinned host->device upload of the inputs and the device->host read of the sampled tokens.
Also reported: decode tok/s per user at batch 1 and the p50 time to first token of a 2048-token prompt.
Weights are random-init N(0, 0.02) quantised to NVFP4, prompts are uniform-random token ids (synthetic).
Each step streams all weights and the whole KV (tens of GB), far larger than L2, so no explicit flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REF_UNAVAILABLE = ("reference installs offline only with --no-deps and cannot run here: it serves pinned "
                   "HF checkpoints (no network), refuses non-GB10 hosts, needs torch>=2.13 + flashinfer 0.6.17 + "
                   "b12x (absent) and JIT-builds sm_121a-only kernels")
# The reference publishes no number for this configuration (BASELINE.json "published" is empty); its closest figure
# is a different model on different hardware and is reported as context only, never as a ratio.
GB10_CONTEXT = {"tok_s": 165.0, "what": "reference hybrid 27B, 4 speculative requests, aggregate, 1x GB10",
                "source": "docs/operations.md:220"}


def _clock_sampler():
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
        return None


def _clock_summary(proc, gpu_index: int) -> dict:
    if proc is None:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    proc.terminate()
    try:
        out, _ = proc.communicate(timeout=5)
    except Exception:  # noqa: BLE001
        proc.kill()
        out = ""
    sm, mx, reasons = [], [], set()
    for line in out.splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 9 or not f[0].isdigit() or int(f[0]) != gpu_index:
            continue
        try:
            sm.append(float(f[1]))
            mx.append(float(f[2]))
        except ValueError:
            continue
        for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
            if val.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm)}


def hybrid_config(args) -> None:
    """Configs 4 and 5: the full-depth hybrid MoE families through `LLM` (hibana_b200/profiling/bench_config.py),
    reported in this file's line format."""
    from hibana_b200.profiling import bench_config
    family = {4: "flashnext", 5: "nemotron"}[args.config]
    batch = args.batch if args.batch != 64 else {4: 32, 5: 16}[args.config]
    prompt = args.prompt if args.prompt != 2048 else {4: 4096, 5: 8192}[args.config]
    argv = ["--family", family, "--mode", args.mode, "--batch", str(batch), "--prompt", str(prompt),
            "--steps", str(args.steps), "--warmup", str(max(args.warmup, 3))]
    if args.layers:
        argv += ["--layers", str(args.layers)]
    out = bench_config.main(argv, emit=None)
    if out is None:
        return
    world = out["n_gpus"]
    print(json.dumps({
        "metric": f"aggregate decode tok/s ({family} hybrid MoE NVFP4, batch {batch}, {prompt} in); also tok/s/user",
        "value": out.get("tok_s", out["tok_s_e2e"]), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": out.get("ms_per_step", out["ms_per_step_e2e"]),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 weights, bf16 activations",
        "data": out["data"],
        "config": {"model": family, "layers": out["layers"], "global_batch": batch, "seq_len": prompt,
                   "parallelism": f"{out['mode']}{world}" if world > 1 else "single", "valid": out["valid"],
                   "l2": "each step streams the routed experts' weights and the KV / state pools (larger than L2)"},
        "e2e": {"value": out["tok_s_e2e"], "unit": "tok/s", "ms_per_step": out["ms_per_step_e2e"]},
        "decode_tok_s_per_user": out.get("tok_s_per_user", out["tok_s_per_user_e2e"]),
        "prefill_ms_per_chunk": out["prefill_ms_per_chunk"], "launches_per_step": out["launches_per_step"],
        "gpu_launches": out["launches_per_step"] * args.steps, "device_status": out["device_status"]}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the result invalid)")
    ap.add_argument("--no-extras", action="store_true", help="skip the batch-8, NCCL-only and token-hash extras")
    ap.add_argument("--config", type=int, default=2, choices=(2, 4, 5),
                    help="2: 27B dense (the headline, default); 4: Flash-Next-class hybrid MoE; 5: Nemotron-class hybrid MoE")
    ap.add_argument("--mode", default="tp", choices=("tp", "dpep"),
                    help="configs 4 and 5 on several GPUs: tensor parallel, or data-parallel replicas + expert parallel")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return
    if args.config != 2:
        return hybrid_config(args)

    import torch
    import torch.distributed as dist

    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import Request, SamplingParams, State
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_27b, scaled

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from hibana_b200.parallel.comm import Communicator
        comm = Communicator.create(rank, world, dev, slot_mb=32, sp_rows=args.prompt, sp_hidden=5120)
    warmup = max(args.warmup, 3)
    steps = args.steps

    t = dense_27b()
    if args.layers:
        t = scaled(t, layers=args.layers)
    tp = world
    t_rank = t.shard(tp, rank)
    model = DenseModel(t_rank, dev, seed=0) if tp == 1 else DenseModel.sharded(t, tp, rank, dev, seed=0)
    batch, prompt_len = args.batch, args.prompt
    max_ctx = prompt_len + warmup + steps + 80
    ex = Executor(model, max_batch=batch, max_ctx=max_ctx, kv_slots=batch * max_ctx + 4096, use_graphs=True,
                  buckets=tuple(sorted({1, min(8, batch), batch})), comm=comm)

    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, t.vocab, (prompt_len,), generator=g).tolist() for _ in range(batch)]

    # Static activation scales from one calibration forward over a short random prompt.
    def calib():
        r = Request(prompt_ids=prompts[0][:256], params=SamplingParams(max_tokens=1))
        ex.admit(r)
        ex.prefill_batch([(r, 256)])
        ex.release(r)
    model.calibrate(calib, comm)

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

    # ---- time to first token: one 2048-token prompt on an idle engine, 3 warm-up + 5 timed
    ttfts = []
    for i in range(8):
        r = Request(prompt_ids=prompts[i % batch], params=SamplingParams(max_tokens=1))
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ex.admit(r)
        ex.prefill_batch([(r, prompt_len)])
        e1.record()
        torch.cuda.synchronize()
        ex.release(r)
        if i >= 3:
            ttfts.append(max_over_ranks(e0.elapsed_time(e1)))
    ttft_p50 = statistics.median(ttfts)

    ex.capture_graphs()

    def run_decode(nreq: int):
        """Prefills nreq prompts, then returns (device ms/step over graph replays, e2e ms/step, clocks)."""
        reqs = [Request(prompt_ids=prompts[i], params=SamplingParams(max_tokens=10 ** 6, ignore_eos=True))
                for i in range(nreq)]
        for r in reqs:
            ex.admit(r)
        for i in range(0, nreq, 2):
            ex.prefill_batch([(r, prompt_len) for r in reqs[i:i + 2]])
        for _ in range(warmup):
            ex.decode_step(reqs)
        torch.cuda.synchronize()
        code = nv.read_status(dev)
        if code != 0:       # a bounded wait ran out in some kernel: every further step would pay its limit again
            raise SystemExit(f"device status {code} after warm-up; not timing a failing run")
        # e2e: public API, upload + graph + readback every step
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h2d0, d2h0 = ex.runner.h2d_bytes, ex.runner.d2h_bytes
        w0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            ex.decode_step(reqs)
        e1.record()
        sync_all()
        wall_ms = (time.perf_counter() - w0) * 1e3 / steps
        e2e_ms = max_over_ranks(max(e0.elapsed_time(e1) / steps, wall_ms))
        h2d = (ex.runner.h2d_bytes - h2d0) / steps
        d2h = (ex.runner.d2h_bytes - d2h0) / steps
        # device-timed: K replays of the captured step (inputs left on the device from the last step); with tensor
        # parallelism that is the greedy step (per-rank argmax + pair exchange), the one decode_step replays here
        buf = ex.runner.bufs[ex.runner._bucket(nreq)]
        graph = buf.graph_greedy if getattr(buf, "graph_greedy", None) is not None else buf.graph
        sync_all()
        proc = _clock_sampler() if rank == 0 else None
        time.sleep(0.3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        sync_all()
        dev_ms = max_over_ranks(e0.elapsed_time(e1) / steps)
        clocks = _clock_summary(proc, local) if rank == 0 else {}
        for r in reqs:
            ex.release(r)
        return dev_ms, e2e_ms, h2d, d2h, clocks

    calls0 = nv.CALLS
    dev1, e2e1, _, _, _ = run_decode(1)
    devb, e2eb, h2d, d2h, clocks = run_decode(batch)
    status = nv.read_status(dev)
    launches_per_step = getattr(ex.runner, "graph_launches", {}).get(batch, 0)
    extras = {}
    if not args.no_extras:
        import hashlib
        dev8, e2e8, _, _, _ = run_decode(min(8, batch))
        extras["decode_tok_s_per_user_b8"] = round(1e3 / dev8, 1)
        # greedy tokens of a short fixed prompt: the same request on every GPU count (tensor-parallel sums round
        # differently, so later tokens may legitimately differ between N; the head and the hash make that visible)
        out = ex.generate_batch([prompts[0][:64]], SamplingParams(max_tokens=16, ignore_eos=True))[0].output_ids
        extras["tokens_head"] = out[:8]
        extras["token_hash"] = hashlib.sha1(",".join(map(str, out)).encode()).hexdigest()[:12]

        def first_token_logprobs():
            """Top-8 (token, logprob) of the first generated token of the fixed prompt (prefill path)."""
            r = ex.generate_batch([prompts[0][:64]], SamplingParams(max_tokens=1, ignore_eos=True, logprobs=8))[0]
            return dict(r.token_logprobs[0][1]) if r.token_logprobs else {}
        fused_lp = first_token_logprobs()
        if comm is not None:
            # same model, same engine, collectives through NCCL only (the unfused baseline on this box)
            comm.fused = False
            for b_ in ex.runner.bufs.values():
                b_.graph = None
                b_.graph_greedy = None
            split = ex.runner._split_head
            ex.runner._split_head = lambda: False
            ex.capture_graphs()
            devn, _, _, _, _ = run_decode(batch)
            extras["nccl_only"] = {"value": round(batch / devn * 1e3, 1), "unit": "tok/s", "ms_per_step": round(devn, 4)}
            # the hand-written collectives against NCCL on the run itself: the same prompt through both, compared on
            # the log-probabilities of the first token (a wrong sum in a fused kernel shows up here, not only as a
            # status word)
            nccl_lp = first_token_logprobs()
            common = set(fused_lp) & set(nccl_lp)
            extras["fused_vs_nccl"] = {
                "top8_tokens_in_common": len(common),
                "max_abs_logprob_diff": round(max((abs(fused_lp[k] - nccl_lp[k]) for k in common), default=-1.0), 5)}
            ex.runner._split_head = split
            comm.fused = True

    if rank == 0:
        value = batch / devb * 1e3
        res = {
            "metric": "aggregate decode tok/s (27B-class dense NVFP4, batch 64, 2048 in); also tok/s/user and p50 TTFT",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(devb, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "gb10_context": GB10_CONTEXT, "dtype": "nvfp4 weights, bf16 activations/KV",
            "data": "synthetic (uniform-random token ids, random-init N(0,0.02) weights quantised to NVFP4)",
            "config": {"model": t.name, "layers": len(t.layers), "global_batch": batch, "seq_len": prompt_len,
                       "parallelism": f"tp{tp}", "context_during_timed_steps": f"{prompt_len}+",
                       "l2": "each step streams >40 GB of weights+KV (inputs larger than L2)",
                       "valid": not args.layers},
            "decode_tok_s_per_user_b1": round(1e3 / dev1, 1),
            "ttft_p50_ms": round(ttft_p50, 2),
            "e2e": {"value": round(batch / e2eb * 1e3, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "tok_s_per_user_b1": round(1e3 / e2e1, 1)},
            "gpu_launches": int(launches_per_step * steps), "launches_per_step": int(launches_per_step),
            "clocks": clocks, "device_status": status, "native_calls_total": nv.CALLS - calls0,
            "kv_bytes_per_token": int(ex.kv.bytes_per_token) * world,
        }
        res.update(extras)
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)   # NCCL teardown with peer-mapped heaps alive can hang; the measurement is already printed


if __name__ == "__main__":
    main()
