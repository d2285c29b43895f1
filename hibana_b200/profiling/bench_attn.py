"""Attention micro-benchmark: python -m hibana_b200.profiling.bench_attn [--mode prefill|decode] ...

prefill: `--batch` sequences of `--rows` new tokens on top of `--prefix` cached tokens; reports TFLOP/s of the causal
         work (4 * D * visible (query, key) pairs per query head) against the measured bf16 GEMM peak.
decode : one token per sequence at context `--ctx`; reports KV bytes / time against the measured copy bandwidth.
The KV pool is token-granular; slots ascend per sequence as a fresh pool hands them out (--shuffled: random order).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch

from .. import config as cfgmod
from ..ops import attention
from .timing import measured_peaks, time_cuda


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="prefill")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--prefix", type=int, default=0)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=40)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shuffled", action="store_true", help="random slot order (worst case: every row is gathered)")
    ap.add_argument("--slot-major", action="store_true", help="pool stored [slots, heads, D] instead of head-major")
    ap.add_argument("--roles", action="store_true", help="prefill: cycles per tile each kernel role spends waiting")
    ap.add_argument("--once", action="store_true", help="single launch, no timing loop (for ncu)")
    args = ap.parse_args()
    dev = torch.device("cuda")
    peaks = measured_peaks()
    b, hq, hkv, d = args.batch, args.hq, args.hkv, args.d
    if args.mode == "prefill":
        rows, ctx_n = args.rows, args.prefix + args.rows
    else:
        rows, ctx_n = 1, args.ctx
    slots = b * ctx_n + 1
    if args.slot_major:
        kp = torch.randn(slots, hkv, d, device=dev).bfloat16()
        vp = torch.randn(slots, hkv, d, device=dev).bfloat16()
    else:       # the engine's pools: head-major storage behind a [slots, heads, D] view
        kp = torch.randn(hkv, slots, d, device=dev).bfloat16().transpose(0, 1)
        vp = torch.randn(hkv, slots, d, device=dev).bfloat16().transpose(0, 1)
    if args.shuffled:
        perm = (torch.randperm(slots - 1, device=dev) + 1).int()
    else:       # ascending runs per sequence, as the pool hands them out to a prefill
        perm = torch.arange(1, slots, device=dev).int()
    idx = perm.view(b, ctx_n).contiguous()
    ctx = torch.full((b,), ctx_n, dtype=torch.int32, device=dev)
    q = torch.randn(b * rows, hq, d, device=dev).bfloat16()
    out = torch.empty_like(q)
    if args.mode == "prefill":
        indptr = (torch.arange(b + 1, device=dev) * rows).int()
        fn = lambda: attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=rows, out=out)  # noqa
        pairs = b * (rows * args.prefix + rows * (rows + 1) // 2)
        flops = 4.0 * d * pairs * hq
    else:
        splits = attention.choose_splits(b, hkv, ctx_n)
        ws = attention.AttnWorkspace(b, hq, d, splits, dev)
        fn = lambda: attention.paged_attention(q, kp, vp, idx, ctx, splits=splits, workspace=ws, out=out)  # noqa
        flops = 4.0 * d * b * ctx_n * hq
    kv_bytes = 2.0 * b * ctx_n * hkv * d * 2
    if args.once:
        fn()
        torch.cuda.synchronize()
        return
    # decode: bursts of 20 launches per sample when the KV read per launch exceeds L2 (see time_cuda)
    burst = 20 if args.mode == "decode" and kv_bytes > 256e6 else 1
    t = time_cuda(fn, iters=args.iters, burst=burst)
    ms = t["median_ms"]
    roles = None
    if args.roles and args.mode == "prefill":
        from .. import _native as nv
        buf = torch.zeros(16, dtype=torch.int64, device=dev)
        nv.lib().hb_attn_prefill_profile(ctypes.c_void_p(buf.data_ptr()))
        fn()
        torch.cuda.synchronize()
        nv.lib().hb_attn_prefill_profile(None)
        c = buf.tolist()
        tiles = max(c[11], 1)
        names = {0: "softmax_wait_scores", 1: "softmax_wait_prev_pv", 3: "issuer_wait_p", 4: "issuer_wait_v",
                 5: "issuer_wait_k", 6: "producer_wait_k_stage", 7: "producer_wait_v_stage", 8: "producer_issue",
                 9: "producer_wait_landed", 10: "softmax_loop_total", 12: "softmax_load_scores",
                 13: "softmax_math", 14: "softmax_publish"}
        roles = {v: round(c[k] / tiles) for k, v in names.items()}
    res = {"mode": args.mode, "batch": b, "rows": rows, "ctx": ctx_n, "hq": hq, "hkv": hkv, "d": d,
           "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "kv_gbs": round(kv_bytes / ms / 1e6, 1),
           "peaks": peaks["source"]}
    if args.mode == "prefill":
        res["frac_of_bf16_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 3)
    else:
        res["frac_of_hbm"] = round(kv_bytes / ms / 1e6 / peaks["hbm_gbs"], 3)
    if args.roles and args.mode == "decode" and d == 128 and cfgmod.current().decode_attn == "tc":
        prof = attention.DecodeTcProfile(dev)
        fn()
        res["tc_cycles_per_tile"] = prof.read()
        prof.close()
    elif args.roles and args.mode == "decode":
        from .. import _native as nv
        buf = torch.zeros(8, dtype=torch.int64, device=dev)
        nv.lib().hb_attn_decode_profile(ctypes.c_void_p(buf.data_ptr()))
        fn()
        torch.cuda.synchronize()
        nv.lib().hb_attn_decode_profile(None)
        c = buf.tolist()
        tiles, ctas = max(c[5], 1), max(c[6], 1)
        res["warp0_cycles"] = {"issue_per_tile": round(c[0] / tiles), "wait_per_tile": round(c[1] / tiles),
                               "math_per_tile": round(c[2] / tiles), "loop_per_cta": round(c[3] / ctas),
                               "merge_per_cta": round(c[4] / ctas), "tiles_per_cta_warp": round(tiles / ctas, 1)}
    if roles is not None:
        res["cycles_per_tile"] = roles
    print(json.dumps(res))


if __name__ == "__main__":
    main()
