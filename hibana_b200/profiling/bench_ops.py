"""Micro-benchmarks of the op kernels that are not GEMMs or attention: python -m hibana_b200.profiling.bench_ops

One JSON line per op: CUDA-event time (median over samples of `--burst` back-to-back launches, L2 flushed between
samples), the algorithmic bytes the op has
to move and the fraction of the measured copy rate that is. Shapes are the 27B / Flash-Next / Nemotron geometries at
a prefill chunk (2048 rows) and at a decode batch (64 rows); latency-bound decode kernels report microseconds, the
fraction is there to show how far from the stream they are. `--only name` runs one op.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..cache.state_pool import StatePool
from ..ops import basic, fp8, moe, nvfp4, recurrent, sampling, ssm_window
from .timing import measured_peaks, time_cuda


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--burst", type=int, default=8,
                    help="back-to-back launches per sample (a lone launch from an idle GPU carries ~20 us of launch "
                         "latency); working sets smaller than L2 are then partly served from L2")
    args = ap.parse_args()
    dev = torch.device("cuda")
    peaks = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).bfloat16()

    ops = []

    def op(name, nbytes, fn):
        ops.append((name, nbytes, fn))

    h = 5120
    for rows in (2048, 64):
        x, res, w = rnd(rows, h), rnd(rows, h), rnd(h).abs()
        gs = torch.tensor(8.0 / (6 * 448), device=dev)
        op(f"rmsnorm+residual rows={rows} h={h}", rows * h * 2 * 4, lambda x=x, res=res, w=w: basic.rmsnorm(x, w, 1e-6, residual=res))
        op(f"norm+quant nvfp4 rows={rows} h={h}", rows * h * (2 * 3 + 0.5625),
           lambda x=x, res=res, w=w: nvfp4.rmsnorm_quantize(x, w, 1e-6, gs, residual=res))
        op(f"quant nvfp4 rows={rows} k=17408", rows * 17408 * (2 + 0.5625),
           lambda a=rnd(rows, 17408): nvfp4.quantize(a, gs))
        op(f"silu-mul rows={rows} inter=17408", rows * 17408 * 2 * 3,
           lambda a=rnd(rows, 2 * 17408): basic.act_mul(a, basic.ACT_SILU_PAIRS))
        op(f"quant fp8 rows rows={rows} h={h}", rows * h * 3, lambda a=x: fp8.quantize_rows(a))
    # RoPE + KV write (27B: 40 q / 8 kv heads x 128)
    for rows in (2048, 64):
        hq, hkv, d = 40, 8, 128
        qkv = rnd(rows, (hq + 2 * hkv) * d)
        pos = torch.arange(rows, dtype=torch.int32, device=dev)
        slots = torch.arange(1, rows + 1, dtype=torch.int32, device=dev)
        inv = basic.rope_inv_freq(d, 1e6).to(dev)
        kp = torch.zeros(rows + 8, hkv, d, dtype=torch.bfloat16, device=dev)
        vp = torch.zeros_like(kp)
        from types import SimpleNamespace

        def rope(qkv=qkv, pos=pos, slots=slots, kp=kp, vp=vp):
            ctx = SimpleNamespace(positions=pos, extras={})
            return basic.rope_kv_write(qkv, pos, slots, inv, kp, vp, hq, hkv, d, table=basic.rope_table(ctx, inv, d))
        op(f"rope+kv write rows={rows} 40q/8kv x128 (with its angle table)", rows * (hq + 2 * hkv) * d * 2 * 2, rope)
    # Mamba-2 decode scan, Nemotron geometry (128 heads x 64 x 128, 8 groups), batch 64: fp32 / int8 / window records
    heads, groups, p, n, b = 128, 8, 64, 128, 64
    xs, bm, cm, dtv = rnd(b, heads * p, scale=0.5), rnd(b, groups * n, scale=0.3), rnd(b, groups * n, scale=0.3), rnd(b, heads, scale=0.5)
    a_log = torch.zeros(heads, device=dev)
    slot = torch.arange(1, b + 1, dtype=torch.int32, device=dev)
    for name, dtype, window, per_state in (("fp32", torch.float32, 0, 8.0), ("int8", torch.int8, 0, 2.0),
                                           ("int8 window records", torch.int8, 16, 1.0)):
        pool = StatePool(1, b + 1, 8, 4, (heads, p, n), dev, state_dtype=dtype, window=window, groups=groups)
        if window:
            ws = pool.window_state(0)
            fn = lambda ws=ws: ssm_window.step(ws, xs, bm, cm, dtv, a_log, None, None, slot)     # noqa: E731
        else:
            fn = lambda pool=pool: recurrent.mamba2_scan(xs, bm, cm, dtv, a_log, None, None, pool.ssm[0], slot, slot,   # noqa: E731
                                                         heads=heads, groups=groups, head_dim=p, d_state=n,
                                                         state_scale=pool.ssm_scale[0] if pool.ssm_scale is not None else None)
        op(f"mamba2 decode scan batch={b} 128h x 64 x 128, state {name}", b * heads * p * n * per_state, fn)
    # gated delta rule decode, Flash-Next geometry (16 k / 48 v heads x 128), batch 32
    b, kh, vh, kd = 32, 16, 48, 128
    q_, k_, v_ = rnd(b, kh * kd, scale=0.3), rnd(b, kh * kd, scale=0.3), rnd(b, vh * kd, scale=0.3)
    gg, beta = torch.rand(b, vh, generator=g, device=dev) * -0.1, torch.rand(b, vh, generator=g, device=dev)
    gpool = StatePool(1, b + 1, 8, 4, (vh, kd, kd), dev)
    gslot = torch.arange(1, b + 1, dtype=torch.int32, device=dev)
    op(f"gated delta rule decode batch={b} 48 v-heads x 128 x 128 fp32", b * vh * kd * kd * 8,
       lambda: recurrent.gdn_scan(q_, k_, v_, gg, beta, gpool.ssm[0], gslot, gslot, k_heads=kh, v_heads=vh, kdim=kd,
                                  vdim=kd, l2norm=True))
    # routing and planning (512 experts)
    for rows, k in ((64, 22), (2048, 10)):
        lg = torch.randn(rows, 512, generator=g, device=dev)
        op(f"route rows={rows} top-{k} of 512", rows * 512 * 4, lambda lg=lg, k=k: moe.route(lg, k, sigmoid=True, renorm=True))
    # sampling over the 27B vocabulary
    lg = torch.randn(64, 151936, generator=g, device=dev)
    op("argmax rows=64 vocab=151936", 64 * 151936 * 4, lambda: sampling.argmax(lg))
    # weight formats beside NVFP4 at a decode batch: FP8 (tcgen05 kind::f8f6f4), 3-bit (dequantisation fused into the
    # GEMM), GGML IQ2_XXS (decode fused into the GEMV)
    from ..ops import ggml as ggml_ops
    from ..ops.w3gemm import W3Linear
    wm, wn, wk = 64, 5120, 17408
    xa = rnd(wm, wk)
    wf = fp8.Fp8Weight.quantize(rnd(wn, wk, scale=0.02))
    xq8, xs8 = fp8.quantize_rows(xa)
    op(f"fp8 GEMM {wm} x {wn} x {wk}", wn * wk, lambda: fp8.linear_fp8(xq8, wf, row_scales=xs8))
    w3 = W3Linear.from_weight(rnd(wn, wk, scale=0.02).float().cpu(), dev, keep_codes=False)
    op(f"3-bit GEMM {wm} x {wn} x {wk} (codes + scale / zero per 64)", wn * wk * (3 / 8 + 4 / 64), lambda: w3(xa))
    gn, gk = 4096, 4096
    grid = (torch.arange(256 * 8, dtype=torch.int64) % 3 * 8 + 1).view(256, 8).to(torch.uint8)
    pl = ggml_ops.PackedLinear(ggml_ops.random_blocks("iq2_xxs", gn, gk, seed=1).to(dev), "iq2_xxs", gn, gk, grid)
    x1 = rnd(1, gk)
    op(f"GGML IQ2_XXS GEMV 1 x {gn} x {gk}", gn * gk * 66 / 256, lambda: pl(x1))
    q8 = ggml_ops.PackedLinear(ggml_ops.random_blocks("q8_0", gn, gk, seed=2).to(dev), "q8_0", gn, gk)
    op(f"GGML Q8_0 GEMV 1 x {gn} x {gk}", gn * gk * 34 / 32, lambda: q8(x1))
    # SSD tier gather: 256 token rows of all layers of a 27B-shaped bf16 KV pool into one staging buffer
    from ..cache.kv_pool import KvPool
    kvp = KvPool(64, 4096, 8, 128, torch.bfloat16, dev)
    ids = torch.randperm(4000, device=dev)[:256].int() + 1
    stage = torch.empty(256 * kvp.bytes_per_token, dtype=torch.uint8, device=dev)
    op("kv gather 256 tokens x 64 layers (pool -> staging)", 2 * 256 * kvp.bytes_per_token,
       lambda: kvp.copy_payload(ids, stage, to_pool=False))
    # hyper-connection site at Flash-Next width
    from ..models.hyper import HyperConnection
    hc_, hh_, rk_ = 4, 2560, 320
    site = HyperConnection(torch.zeros(hc_ * hh_, device=dev), rnd(rk_, hc_ * hh_, scale=0.02), rnd(hc_ * hh_, rk_, scale=0.02),
                           rnd(hc_, hc_ * hh_, scale=0.02), hc_, hh_)
    hyp, blk = rnd(32, hc_ * hh_), rnd(32, hh_)

    def hyper_site():
        mixed, keep = site.mix(hyp)
        return site.combine(blk, keep)
    op("hyper-connection mix + combine, 32 rows x 4 streams x 2560 (6 launches)",
       (rk_ + 16 + hc_ * hh_) * hc_ * hh_ * 2 * 0 + (site.down_inject.numel() + site.up.numel()) * 2, hyper_site)
    # routed experts at a decode batch, Nemotron geometry (512 experts, 1024 -> 2688 -> 1024, squared ReLU, top-22,
    # 16 rows): the served NVFP4 stacks against the 3-bit decode copy (grouped GEMMs, dequantisation fused). Built
    # only when asked for by name: the stacks take a few GB.
    if args.only and args.only in "routed experts":
        e_, hid_, inter_, rows_, topk_ = 512, 1024, 2688, 16, 22
        fc1, fc2 = rnd(e_, inter_, hid_, scale=0.02), rnd(e_, hid_, inter_, scale=0.02)
        xe = rnd(rows_, hid_)
        eids = torch.stack([torch.randperm(e_, generator=g, device=dev)[:topk_] for _ in range(rows_)]).int()
        ew_ = torch.softmax(torch.randn(rows_, topk_, generator=g, device=dev), -1)
        distinct = int(eids.unique().numel())
        per_expert = 2 * inter_ * hid_
        for fmt_, bits in (("nvfp4", 4.5), ("w3", 4.0)):
            ew = moe.ExpertWeights.create(fc1, fc2, "relu2", fmt_).to(dev)
            op(f"routed experts {rows_} rows top-{topk_} of {e_} ({distinct} distinct), 1024-2688-1024, {fmt_} stacks",
               distinct * per_expert * bits / 8, lambda ew=ew: moe.experts_forward(xe, eids, ew_, ew))
        del fc1, fc2
    for name, nbytes, fn in ops:
        if args.only and args.only not in name:
            continue
        t = time_cuda(fn, iters=args.iters, burst=args.burst)
        ms = t["median_ms"]
        gbs = nbytes / ms / 1e6
        print(json.dumps({"op": name, "us": round(ms * 1e3, 1), "algorithmic_mb": round(nbytes / 1e6, 2),
                          "gbs": round(gbs, 1), "of_measured_copy_rate": round(gbs / peaks["hbm_gbs"], 3),
                          "peaks": peaks["source"]}), flush=True)


if __name__ == "__main__":
    main()
