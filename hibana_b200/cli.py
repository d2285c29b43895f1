"""`hibana` command line: serve | chat | status | stop | cache | logs | launch | traces | verify | engine | dev |
gate | h2h | eval | cache-trace.

`serve` resolves settings and runs the server in the foreground (with --tp/--dp > 1 under the rank supervisor);
`launch` does the same detached; `engine` is the per-rank entry the supervisor spawns; `dev` hosts the
micro-benchmarks. Reference: hibana/cli.py:33-298.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional


def add_engine_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("target", nargs="?", default=None)
    p.add_argument("--profile", choices=("exact", "fast", "throughput"))
    p.add_argument("--config-file")
    p.add_argument("--host")
    p.add_argument("--port", type=int)
    p.add_argument("--tp", type=int, choices=(1, 2, 4, 8))
    p.add_argument("--ep", type=int, choices=(1, 2, 4, 8))
    p.add_argument("--dp", type=int, choices=(1, 2, 4, 8))
    p.add_argument("--max-batch", type=int, dest="max_batch")
    p.add_argument("--max-context", type=int, dest="max_context")
    p.add_argument("--weights")
    p.add_argument("--spec", choices=("off", "mtp", "dflash2", "ngram", "lilicorr"))
    p.add_argument("--spec-depth", type=int, dest="spec_depth")
    p.add_argument("--ssd-dir", dest="ssd_dir")
    p.add_argument("--w3", action="store_const", const=True, dest="w3", help="3-bit decode copies beside the weights")
    p.add_argument("--w3-checkpoint", dest="w3_checkpoint", help="calibrated 3-bit copies (weights/calibrate_model.py)")
    p.add_argument("--kv-dtype", dest="kv_dtype", choices=("bf16", "fp8", "nvfp4"))
    p.add_argument("--ssm-state", dest="ssm_state", choices=("fp32", "fp16_sr", "int8", "int8w"))
    p.add_argument("--no-graphs", action="store_const", const=False, dest="cuda_graphs")
    p.add_argument("--no-fused-collectives", action="store_const", const=False, dest="fused_collectives")
    p.add_argument("--trace-dir", dest="trace_dir")


def _flags(args) -> dict:
    keys = ("host", "port", "tp", "ep", "dp", "max_batch", "max_context", "weights", "spec", "spec_depth", "ssd_dir",
            "cuda_graphs", "fused_collectives", "trace_dir", "w3", "w3_checkpoint", "kv_dtype", "ssm_state")
    return {k: getattr(args, k, None) for k in keys}


def _resolve(args):
    from .launch.settings import resolve
    return resolve(args.target, profile=args.profile, config_file=args.config_file, flags=_flags(args))


def run_engine(args) -> int:
    """Per-process entry: installs the resolved config, joins the process group when WORLD_SIZE > 1, serves."""
    from . import config as cfgmod
    cfg = _resolve(args)
    cfgmod.install(cfg)
    from .launch import preflight
    host = preflight.check_host(need_gpus=max(cfg.tp * cfg.dp, 1), require_b200=False)
    for problem in host.problems:
        print("preflight:", problem, file=sys.stderr)
    try:
        weights = preflight.ensure_weights(cfg, fetch=not getattr(args, "no_fetch", False))
        w3_dir = preflight.ensure_w3(cfg)
    except preflight.PreflightError as e:
        raise SystemExit(f"preflight: {e}") from None
    if weights is not None:
        cfg = cfg.replace(weights=str(weights))
    if int(os.environ.get("RANK", "0")) == 0:
        print(preflight.summary(cfg, host, weights, w3_dir), file=sys.stderr)
    if cfg.host_floor_gib > 0 and int(os.environ.get("LOCAL_RANK", "0")) == 0:
        # one guard per host: under sustained host-memory pressure it asks this process to stop (the supervisor of
        # a rank group then restarts or gives up by its policy) instead of letting the kernel's OOM killer choose
        from .launch.guard import MemoryGuard
        MemoryGuard(cfg.host_floor_gib).start()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        from .parallel.lockstep import serve_rank
        return serve_rank(cfg)
    from .api.server import serve
    serve(cfg)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="hibana", description="Blackwell-native LLM inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("serve", "engine", "launch"):
        add_engine_args(sub.add_parser(name))
    for name in ("status", "stop", "cache", "verify", "chat"):
        p = sub.add_parser(name)
        p.add_argument("--host", default="127.0.0.1")
        p.add_argument("--port", type=int, default=30001)
        if name == "cache":
            p.add_argument("--flush", action="store_true")
        if name == "chat":
            p.add_argument("--max-tokens", type=int, default=256)
    p = sub.add_parser("logs")
    p.add_argument("--port", type=int, default=30001)
    p.add_argument("-n", type=int, default=40)
    p = sub.add_parser("traces")
    p.add_argument("--dir", required=True)
    for name in ("gate", "h2h", "eval"):         # quality / speed tooling (hibana_b200/evals): arguments pass through
        sub.add_parser(name, add_help=False).add_argument("rest", nargs=argparse.REMAINDER)
    p = sub.add_parser("cache-trace")
    p.add_argument("target", nargs="?", default="dense-tiny")
    p.add_argument("--tokens", type=int, default=96)
    p.add_argument("--prefix", type=int, default=64)
    p.add_argument("--out", default="cache_trace.json")
    p = sub.add_parser("dev")
    p.add_argument("tool", choices=("bench-gemm", "bench-attn", "tp-comm", "build", "check-host"))
    p.add_argument("rest", nargs=argparse.REMAINDER)
    return ap


def main(argv: Optional[list] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.cmd == "engine":
        return run_engine(args)
    if args.cmd == "serve":
        cfg = _resolve(args)
        if cfg.tp * cfg.dp > 1:
            from .launch.supervisor import RankGroup, Supervisor, engine_argv
            extra = [a for a in (sys.argv[2:] if argv is None else argv[1:])]
            return Supervisor(RankGroup(cfg.tp * cfg.dp, engine_argv(extra))).run()
        return run_engine(args)
    if args.cmd == "launch":
        from .launch.service import launch_detached
        cfg = _resolve(args)
        pid = launch_detached(["serve", *(sys.argv[2:] if argv is None else argv[1:])], cfg.port)
        print(json.dumps({"pid": pid, "port": cfg.port}))
        return 0
    if args.cmd in ("gate", "h2h", "eval"):
        from .evals import evaluate, h2h, lossy_gate
        return {"gate": lossy_gate.main, "h2h": h2h.main, "eval": evaluate.main}[args.cmd](args.rest)
    if args.cmd == "cache-trace":
        import pathlib

        import torch

        from . import config as cfgmod
        from .engine import cache_trace
        from .engine.llm import LLM
        cfg = cfgmod.EngineConfig(target=args.target, max_batch=4, cuda_graphs=False, max_context=max(512, 2 * args.tokens))
        llm = LLM(cfg)
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(3, llm.target.vocab, (args.tokens,), generator=g).tolist()
        rep = cache_trace.run(lambda: LLM(cfg, model=llm.model).executor, ids, args.prefix, pathlib.Path(args.out))
        print(json.dumps(rep, indent=1))
        return 0 if all(p["equal"] or p["max_rel_diff"] < 0.05 for p in rep["pairs"].values()) else 1
    from .launch import ctl
    if args.cmd == "status":
        print(json.dumps(ctl.status(args.host, args.port), indent=1, default=str))
        return 0
    if args.cmd == "stop":
        print("stopping" if ctl.stop(args.port) else "not running")
        return 0
    if args.cmd == "cache":
        print(json.dumps(ctl.cache(args.host, args.port, args.flush), indent=1))
        return 0
    if args.cmd == "verify":
        res = ctl.verify(args.host, args.port)
        print(json.dumps(res))
        return 0 if res["ok"] else 1
    if args.cmd == "chat":
        ctl.chat_repl(args.host, args.port, args.max_tokens)
        return 0
    if args.cmd == "logs":
        from .launch.service import log_path
        p = log_path(f"serve-{args.port}")
        print("\n".join(p.read_text(errors="replace").splitlines()[-args.n:]) if p.exists() else f"no log at {p}")
        return 0
    if args.cmd == "traces":
        from .engine.traces import summarize
        print(json.dumps(summarize(args.dir), indent=1))
        return 0
    if args.cmd == "dev":
        if args.tool == "build":
            from . import build_native
            print(build_native.build(verbose=True))
        elif args.tool == "check-host":
            from .launch.preflight import check_host
            rep = check_host()
            print(json.dumps(rep.__dict__, indent=1))
            return 0 if rep.ok else 1
        elif args.tool == "bench-gemm":
            from .profiling import bench_gemm
            sys.argv = ["bench_gemm", *args.rest]
            bench_gemm.main()
        elif args.tool == "bench-attn":
            from .profiling import bench_attn
            sys.argv = ["bench_attn", *args.rest]
            bench_attn.main()
        elif args.tool == "tp-comm":
            from .profiling import tp_comm
            sys.argv = ["tp_comm", *args.rest]
            tp_comm.main()
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
