"""Expert-parallel mixture-of-experts benchmark: fused peer-memory all-to-all vs the NCCL counterpart.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m hibana_b200.profiling.ep_bench

One call = route is given; count -> plan -> dispatch -> grouped fc1 -> act/quant -> grouped fc2 (return epilogue)
-> combine, against all-gather -> local experts over all tokens -> reduce-scatter. Times are CUDA-event medians,
max over ranks. `roof_us` is the slower of (a) the expert weights this rank must stream once from HBM at the
measured copy rate plus the FLOPs at 4x the measured bf16 peak and (b) the bytes that must cross NVLink per
direction at 770 GB/s (NVFP4 rows out, bf16 rows back).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import moe
from ..parallel.ep import ExpertParallel
from .timing import measured_peaks

NVLINK_GBS = 770.0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=512)
    ap.add_argument("--topk", type=int, default=10)
    ap.add_argument("--hidden", type=int, default=2560)
    ap.add_argument("--inter", type=int, default=640)
    ap.add_argument("--tokens", type=int, nargs="*", default=[32, 256, 2048], help="tokens per rank")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--once", action="store_true", help="run the fused call once inside a profiler range, no timing "
                                                        "(for ncu on one GPU)")
    args = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29598")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    e, k, h, inter = args.experts, args.topk, args.hidden, args.inter
    e_per = e // world
    g = torch.Generator().manual_seed(rank)
    fc1 = torch.randn(e_per, 2 * inter, h, generator=g) * 0.03
    fc2 = torch.randn(e_per, h, inter, generator=g) * 0.03
    ew = moe.ExpertWeights.create(fc1.to(dev), fc2.to(dev), "swiglu", "nvfp4")
    del fc1, fc2
    for t in args.tokens:
        ep = ExpertParallel.create(rank, world, dev, tokens=t, topk=k, experts=e, hidden=h)
        x = torch.randn(t, h, device=dev).bfloat16()
        ids, w = moe.route(torch.randn(t, e, device=dev), k)

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(args.iters):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3)
            v = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64, device=dev)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            return float(v.item())

        if args.once:
            for _ in range(2):
                ep.forward(x, ids, w, ew)
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            ep.forward(x, ids, w, ew)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            del ep
            continue
        fused = timed(lambda: ep.forward(x, ids, w, ew))
        nccl = timed(lambda: ep.forward_nccl(x, ids, w, ew))
        pairs = t * k                                    # per rank; on average as many arrive as leave
        remote = pairs * (world - 1) / world
        link_bytes = remote * max(h * 0.5625, h * 2.0)   # per direction: the return (bf16) is the larger leg
        touched = min(e_per, pairs * world // max(world, 1))
        w_bytes = touched * 3 * h * inter * 0.5625
        flops = 2.0 * pairs * 3 * h * inter
        roof = max(w_bytes / (peaks["hbm_gbs"] * 1e3) + flops / (4 * peaks["bf16_tflops"] * 1e6),
                   link_bytes / (NVLINK_GBS * 1e3))
        if rank == 0:
            print(json.dumps({"tokens_per_rank": t, "world": world, "experts": e, "topk": k, "hidden": h,
                              "inter": inter, "fused_us": round(fused, 1), "nccl_us": round(nccl, 1),
                              "speedup": round(nccl / fused, 2), "roof_us": round(roof, 1),
                              "frac_of_roof": round(roof / fused, 3), "peaks": peaks["source"]}), flush=True)
        del ep
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
