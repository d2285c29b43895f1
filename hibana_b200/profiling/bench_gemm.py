"""GEMM micro-benchmark: python -m hibana_b200.profiling.bench_gemm [--kind nvfp4|bf16|gemv] [--shapes m,n,k ...]

`--kind gemv` times the few-row NVFP4 GEMV (ops/gemv.py; `--epi norm` adds its RMSNorm prologue, `--epi silu` the
SiLU-mul epilogue) on the same harness.

Prints one JSON line per shape with the CUDA-event time, achieved TFLOP/s and GB/s and the fraction of the
measured roofline (the slower of FLOPs / bf16 peak and bytes / copy bandwidth), next to torch.matmul (cuBLAS)
on the same bf16 problem for reference.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm, gemv, nvfp4
from .timing import measured_peaks, time_cuda

DEFAULT = ["1,5120,5120", "8,5120,17408", "64,34816,5120", "64,5120,17408", "64,7168,5120", "256,5120,17408",
           "2048,34816,5120", "2048,5120,17408", "8192,7168,5120", "8192,5120,17408"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="nvfp4")
    ap.add_argument("--shapes", nargs="*", default=DEFAULT)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--once", action="store_true", help="single launch per shape, no timing loop (for ncu)")
    ap.add_argument("--graph", action="store_true",
                    help="time a CUDA-graph replay that cycles through weight copies larger than L2 in total")
    ap.add_argument("--pdl", action="store_true", help="launch GEMMs as programmatic dependents")
    ap.add_argument("--phases", action="store_true",
                    help="also print the kernel's phase timers (ns since kernel entry, mean over CTAs)")
    ap.add_argument("--epi", default="store", choices=["store", "silu", "silu_quant", "norm"],
                    help="epilogue (nvfp4): plain store, SiLU-mul, SiLU-mul + NVFP4 requant in the epilogue")
    ap.add_argument("--decode", type=int, default=-1, help="gemv: 0 = cvt, 1 = shift-and-mask code decode")
    args = ap.parse_args()
    gemm.set_pdl(args.pdl)
    if args.decode >= 0:
        from .. import _native as nv
        nv.register("hb_nvfp4_gemv_set_decode", [nv.I], void=True)
        nv.lib().hb_nvfp4_gemv_set_decode(args.decode)
    peaks = measured_peaks()
    dev = torch.device("cuda")
    for spec in args.shapes:
        m, n, k = (int(v) for v in spec.split(","))
        x = torch.randn(m, k, device=dev).bfloat16()
        w = (torch.randn(n, k, device=dev) * 0.02).bfloat16()
        if args.kind == "gemv":
            wq = nvfp4.quantize_weight(w)
            nw = torch.ones(k, dtype=torch.bfloat16, device=dev) if args.epi == "norm" else None
            out = torch.empty(m, n // 2 if args.epi == "silu" else n, dtype=torch.bfloat16, device=dev)

            def run(w_):
                return gemv.nvfp4_gemv(x, w_, norm_weight=nw, out=out,
                                       epilogue=gemm.EPI_SILU_MUL if args.epi == "silu" else gemm.EPI_STORE)
            fn = lambda: run(wq)  # noqa: E731
            bytes_moved = n * k * 0.5625 + m * k * 2 + m * n * 2
        elif args.kind == "nvfp4":
            wq = nvfp4.quantize_weight(w)
            gs = torch.tensor(float(x.float().abs().max()) / (6 * 448), device=dev)
            xq = nvfp4.quantize(x, gs)
            alpha = (gs * wq.gscale).reshape(1)
            out = torch.empty(m, n // 2 if args.epi != "store" else n, dtype=torch.bfloat16, device=dev)
            oscale = torch.tensor(8.0 / (6 * 448), device=dev)

            def run(w_):
                if args.epi == "silu_quant":
                    return gemm.linear_nvfp4_silu_quant(xq, w_, alpha, oscale)
                return gemm.linear_nvfp4(xq, w_, alpha, out=out,
                                         epilogue=gemm.EPI_SILU_MUL if args.epi == "silu" else gemm.EPI_STORE)
            fn = lambda: run(wq)  # noqa: E731
            bytes_moved = n * k * 0.5625 + m * k * 0.5625 + m * n * 2
        else:
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            fn = lambda: gemm.linear_bf16(x, w, out=out)  # noqa: E731
            bytes_moved = (n * k + m * k + m * n) * 2
        if args.once:
            fn()
            torch.cuda.synchronize()
            continue
        if args.graph:
            wbytes = n * k * (0.5625 if args.kind in ("nvfp4", "gemv") else 2)
            reps = min(max(2, int((300 << 20) / wbytes) + 1), 1024)
            if args.kind in ("nvfp4", "gemv"):
                ws = [nvfp4.Nvfp4Tensor(wq.q.clone(), wq.sf.clone(), wq.gscale, wq.rows, wq.k) for _ in range(reps)]
                calls = [lambda w_=w_: run(w_) for w_ in ws]
            else:
                ws = [w.clone() for _ in range(reps)]
                calls = [lambda w_=w_: gemm.linear_bf16(x, w_, out=out) for w_ in ws]
            for c in calls:
                c()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for c in calls:
                    c()
            t = time_cuda(g.replay, iters=args.iters, flush=False)
            t = {"median_ms": t["median_ms"] / reps}
        else:
            t = time_cuda(fn, iters=args.iters)
        phases = None
        if args.phases:
            from .. import _native as nv
            nv.register("hb_gemm_profile", [nv.P], void=True)
            buf = torch.zeros(8, dtype=torch.int64, device=dev)
            nv.lib().hb_gemm_profile(buf.data_ptr())
            for _ in range(20):      # eager launches: the timer buffer is a launch argument, not part of a graph
                fn()
            torch.cuda.synchronize()
            nv.lib().hb_gemm_profile(None)
            c = buf.tolist()
            names = ("setup", "pred_done", "accum_done", "parked", "cluster1", "reduced", "cluster2")
            phases = {n: round(c[i] / max(c[7], 1)) for i, n in enumerate(names)}
        tl = time_cuda(lambda: torch.matmul(x, w.t()), iters=args.iters)
        flops = 2.0 * m * n * k
        ms = t["median_ms"]
        peak_fl = peaks["bf16_tflops"] * (4.0 if args.kind == "nvfp4" else 1.0)

        roof_ms = max(flops / (peak_fl * 1e12), bytes_moved / (peaks["hbm_gbs"] * 1e9)) * 1e3
        print(json.dumps({"kind": args.kind, "m": m, "n": n, "k": k, "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1), "gbs": round(bytes_moved / ms / 1e6, 1),
                          "roofline_frac": round(roof_ms / ms, 3), "cublas_bf16_ms": round(tl["median_ms"], 4), "epi": args.epi,
                          "peaks": peaks["source"], **({"phase_ns": phases} if phases else {})}))


if __name__ == "__main__":
    main()
