"""Tensor-parallel collective benchmark: fused peer-memory kernels vs the NCCL-only path.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m hibana_b200.profiling.tp_comm

Every number is timed on the device with CUDA events around a CUDA-graph replay and is the max over ranks.
  ar_norm   : all-reduce of a [rows, H] bf16 partial + residual add + RMSNorm + NVFP4 quant
              fused = one kernel over NVLink peer loads; nccl = NCCL all-reduce + the local add/norm/quant kernel.
  sp_layer  : the communication-bound half of a prefill layer at M rows: o_proj-shaped row-parallel GEMM ->
              reduce -> norm -> quant -> gate_up-shaped column-parallel GEMM
              fused = GEMM(scatter epilogue) + reduce/norm/all-gather push + flag-gated GEMM
              nccl  = GEMM + NCCL all-reduce + add/norm/quant + GEMM.
Roofline (printed as `roof_us`): the slower of the GEMM FLOPs at 4x the measured bf16 peak and the bytes that must
cross NVLink at 770 GB/s per direction (measured peer-copy rate of this pool).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..models.linear import Linear
from ..ops import gemm, nvfp4
from ..parallel.comm import Communicator
from .timing import measured_peaks

NVLINK_GBS = 770.0


def graph_time(fn, reps: int, iters: int = 5) -> float:
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    best = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best.append(e0.elapsed_time(e1) / reps * 1e3)
    t = torch.tensor([sorted(best)[len(best) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--heads-dim", type=int, default=5120, help="o_proj input width (q heads * head dim), unsharded")
    ap.add_argument("--ffn", type=int, default=17408)
    ap.add_argument("--rows", type=int, nargs="*", default=[1, 16, 64, 256])
    ap.add_argument("--sp-rows", type=int, nargs="*", default=[2048])
    ap.add_argument("--once", action="store_true", help="run each fused op once, no timing (for ncu on one GPU)")
    args = ap.parse_args()
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29599")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    h = args.hidden
    max_sp = max(args.sp_rows) if args.sp_rows else 0
    comm = Communicator.create(rank, world, dev, slot_mb=32, sp_rows=max_sp, sp_hidden=h)
    peaks = measured_peaks()
    out = []
    w = torch.ones(h, dtype=torch.bfloat16, device=dev)
    gs = torch.tensor([8.0 / (6 * 448)], device=dev)
    for rows in args.rows:
        res = torch.randn(rows, h, device=dev).bfloat16()
        slot = 0
        buf = comm.slot_buffer(slot, rows, h)
        buf.copy_(torch.randn(rows, h, device=dev).bfloat16())
        part = buf.clone()

        def fused():
            comm.allreduce_norm(slot, rows, h, residual=res, weight=w, quant_scale=gs, want_bf16=False)

        def nccl():
            dist.all_reduce(part)
            nvfp4.rmsnorm_quantize(part, w, 1e-6, gs, residual=res)
        if args.once:
            for _ in range(2):
                fused()
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            fused()
            nccl()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            continue
        tn = graph_time(nccl, 200)
        was = comm.low_latency
        comm.low_latency = True
        tf = graph_time(fused, 200)          # push protocol (the default only on two ranks)
        comm.low_latency = False
        tflag = graph_time(fused, 200)       # flag-based one-shot (the path larger messages take)
        comm.low_latency = was
        nv_bytes = (world - 1) * rows * h * 2           # one-shot: every rank pulls every peer's partial
        roof = nv_bytes / (NVLINK_GBS * 1e3) if world > 1 else 0.0
        out.append({"op": "ar_norm", "rows": rows, "hidden": h, "world": world, "fused_us": round(tf, 2),
                    "fused_flag_us": round(tflag, 2), "nccl_us": round(tn, 2), "speedup": round(tn / tf, 2), "roof_us": round(roof, 2)})
    # ---- prefill chain
    kin = args.heads_dim // world
    nout = 2 * args.ffn // world
    o_proj = Linear(torch.randn(h, kin, device=dev) * 0.02, "nvfp4").to(dev)
    gate_up = Linear(torch.randn(nout, h, device=dev) * 0.02, "nvfp4").to(dev)
    for m in args.sp_rows:
        if m % (128 * world):
            continue
        x = torch.randn(m, kin, device=dev).bfloat16()
        xq = o_proj.quantize_input(x)
        res_full = torch.randn(m, h, device=dev).bfloat16()
        rpr = m // world
        res_shard = res_full[rank * rpr:(rank + 1) * rpr].contiguous()

        def fused_chain():
            comm.sp_gemm_scatter(o_proj, xq)
            a = comm.sp_reduce_norm_gather(m, h, res_shard, w, 1e-6, quant_scale=gate_up.input_scale)
            comm.sp_gemm_gathered(gate_up, a, epilogue=gemm.EPI_SILU_MUL)

        def nccl_chain():
            part = o_proj(xq)
            dist.all_reduce(part)
            a, _ = nvfp4.rmsnorm_quantize(part, w, 1e-6, gate_up.input_scale, residual=res_full)
            gate_up(a, epilogue=gemm.EPI_SILU_MUL)
        if args.once:
            for _ in range(2):
                fused_chain()
                nccl_chain()
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            fused_chain()
            nccl_chain()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            continue
        tf, tn = graph_time(fused_chain, 20), graph_time(nccl_chain, 20)
        flops = 2.0 * m * h * kin + 2.0 * m * nout * h
        t_math = flops / (peaks["bf16_tflops"] * 4 * 1e12) * 1e6
        nv_bytes = (world - 1) / world * m * h * 2 + (world - 1) * rpr * (h // 2 + h // 16)
        t_link = nv_bytes / (NVLINK_GBS * 1e3)
        out.append({"op": "sp_layer", "rows": m, "world": world, "fused_us": round(tf, 1), "nccl_us": round(tn, 1),
                    "speedup": round(tn / tf, 2), "roof_us": round(max(t_math, t_link), 1),
                    "roof_frac_fused": round(max(t_math, t_link) / tf, 3), "roof_frac_nccl": round(max(t_math, t_link) / tn, 3)})
    comm.check_status()
    if rank == 0:
        for o in out:
            print(json.dumps(o), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
