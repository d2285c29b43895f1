"""Window-record recurrent state (ops/ssm_window.py, csrc/ssm_window.cu): the record stands for the fp32 state it
replaces, a verify pass writes nothing, commits fold once per window, and the engine decodes with it."""
import pytest
import torch

from hibana_b200.cache.state_pool import StatePool
from hibana_b200.ops import recurrent, ssm_window


def _inputs(t, h, g, p, n, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(t, h * p, generator=gen) * 0.5).bfloat16()
    bm = (torch.randn(t, g * n, generator=gen) * 0.3).bfloat16()
    cm = (torch.randn(t, g * n, generator=gen) * 0.3).bfloat16()
    dt = (torch.randn(t, h, generator=gen) * 0.5).bfloat16()
    a_log = torch.log(torch.rand(h, generator=gen) * 4 + 0.5)
    dt_bias = torch.randn(h, generator=gen) * 0.1
    dskip = torch.ones(h)
    return x, bm, cm, dt, a_log, dt_bias, dskip


def _pool(h, g, p, n, window, dev="cpu", slots=6):
    return StatePool(1, slots, 8, 4, (h, p, n), dev, state_dtype=torch.int8, window=window, groups=g)


def test_window_record_tracks_the_fp32_recurrence_cpu():
    h, g, p, n, w = 4, 2, 8, 16, 6
    x, bm, cm, dt, a_log, dt_bias, dskip = _inputs(40, h, g, p, n)
    pool = _pool(h, g, p, n, w)
    ws = pool.window_state(0)
    ref = torch.zeros(7, h, p, n)
    slot = torch.tensor([3], dtype=torch.int32)
    ys, yr = [], []
    for r in range(40):                      # one committing row per call: fresh start, then folds every w rows
        init = torch.tensor([0 if r == 0 else 1], dtype=torch.int32)
        ys.append(ssm_window.step(ws, x[r:r + 1], bm[r:r + 1], cm[r:r + 1], dt[r:r + 1], a_log, dt_bias, dskip, slot,
                                  has_init=init))
        yr.append(recurrent.mamba2_scan(x[r:r + 1], bm[r:r + 1], cm[r:r + 1], dt[r:r + 1], a_log, dt_bias, dskip, ref,
                                        slot, slot, heads=h, groups=g, head_dim=p, d_state=n, has_init=init))
        assert int(ws.win_len[3].max()) <= w            # a call folds before it would exceed the window
    ys, yr = torch.cat(ys).float(), torch.cat(yr).float()
    assert (ys - yr).abs().max() <= 0.03 * yr.abs().max()
    # the record stands for the fp32 state: expansion close to the reference state, quantisation error of int8 rows
    dense = ssm_window.to_dense(ws, slot)[0]
    assert (dense - ref[3]).abs().max() <= 0.03 * ref[3].abs().max()
    # a verify pass (commit=False) over 5 more rows writes nothing and equals the committing replay of the same rows
    before = [t_.clone() for t_ in (ws.z, ws.zscale, ws.win_b, ws.win_u, ws.win_c, ws.win_len)]
    x2, bm2, cm2, dt2, *_ = _inputs(5, h, g, p, n, seed=9)
    ip = torch.tensor([0, 5], dtype=torch.int32)
    v = ssm_window.step(ws, x2, bm2, cm2, dt2, a_log, dt_bias, dskip, slot, q_indptr=ip, commit=False)
    assert all(torch.equal(a, b) for a, b in zip(before, (ws.z, ws.zscale, ws.win_b, ws.win_u, ws.win_c, ws.win_len)))
    c = ssm_window.step(ws, x2[:3], bm2[:3], cm2[:3], dt2[:3], a_log, dt_bias, dskip, slot,
                        q_indptr=torch.tensor([0, 3], dtype=torch.int32))
    # rows of a call that starts with a fold differ from the read-only pass by that fold's quantisation only
    assert (v[:3].float() - c.float()).abs().max() <= 0.03 * v.float().abs().max()
    # from_dense / to_dense round trip and slot bookkeeping
    ssm_window.from_dense(ws, torch.tensor([5], dtype=torch.int32), ref[3:4])
    back = ssm_window.to_dense(ws, torch.tensor([5], dtype=torch.int32))[0]
    assert (back - ref[3]).abs().max() <= 0.01 * ref[3].abs().max() and int(ws.win_len[5].max()) == 0
    pool.copy_slot(3, 1)
    assert torch.equal(pool.win_u[0, 1], pool.win_u[0, 3]) and torch.equal(pool.ssm[0, 1], pool.ssm[0, 3])
    pool.zero_slot(1)
    assert not pool.win_len[0, 1].any() and not pool.ssm[0, 1].any()


def test_engine_decodes_with_window_state_cpu():
    """Tiny hybrid MoE with the int8w state: prefill (dense path), decode, prefix snapshots and speculation run; the
    tokens stay close to the fp32-state run."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import tiny_hybrid_moe
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    pre = torch.randint(0, t.vocab, (40,), generator=g).tolist()
    prompts = [pre + torch.randint(0, t.vocab, (12,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=24)
    ref = [r.output_ids for r in Executor(m, max_batch=4, max_ctx=160, use_graphs=False).generate_batch(prompts, sp)]
    ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, state_dtype=torch.int8, state_window=8)
    assert ex.state_pool.window == 8
    got = [r.output_ids for r in ex.generate_batch(prompts, sp)]
    ex.state.check()
    agree = sum(a == b for x_, y_ in zip(got, ref) for a, b in zip(x_, y_))
    assert [o[0] for o in got] == [o[0] for o in ref] and agree >= 0.6 * 72, agree
    assert int(ex.state_pool.win_len.max()) <= 8 + 16
    spec = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, state_dtype=torch.int8, state_window=8)
    spec.enable_spec(2)
    out = [r.output_ids for r in spec.generate_batch(prompts, sp)]
    spec.state.check()
    agree = sum(a == b for x_, y_ in zip(out, ref) for a, b in zip(x_, y_))
    assert all(len(o) == 24 for o in out) and agree >= 0.5 * 72, agree


@pytest.mark.gpu
@pytest.mark.parametrize("h,g,p,n,w", [(8, 1, 32, 64, 8), (32, 2, 64, 128, 16)])
def test_window_kernel_matches_reference_gpu(h, g, p, n, w):
    """The kernel against the CPU reference of the same arithmetic: single committing rows (with folds), a fresh
    start, multi-row read-only and committing calls, the record tensors themselves, and the dense conversions."""
    from hibana_b200 import _native as nv
    x, bm, cm, dt, a_log, dt_bias, dskip = _inputs(3 * w + 9, h, g, p, n, seed=3)
    cpu, gpu = _pool(h, g, p, n, w), _pool(h, g, p, n, w, "cuda")
    wc, wg = cpu.window_state(0), gpu.window_state(0)
    dev = lambda t_: t_.cuda()       # noqa: E731
    slots = torch.tensor([2, 4], dtype=torch.int32)
    args_c = (a_log, dt_bias, dskip)
    args_g = tuple(dev(a) for a in args_c)

    def both(rows, ip=None, init=None, commit=True, tol=2e-2):
        yc = ssm_window.step(wc, x[rows], bm[rows], cm[rows], dt[rows], *args_c, slots,
                             q_indptr=ip, has_init=init, commit=commit)
        yg = ssm_window.step(wg, dev(x[rows]), dev(bm[rows]), dev(cm[rows]), dev(dt[rows]), *args_g, dev(slots),
                             q_indptr=None if ip is None else dev(ip), has_init=None if init is None else dev(init),
                             commit=commit)
        assert (yg.float().cpu() - yc.float()).abs().max() <= tol * max(yc.float().abs().max().item(), 1e-3)

    r = 0
    both(slice(0, 2), init=torch.tensor([0, 0], dtype=torch.int32))          # fresh slots, one row each
    r = 2
    for _ in range(w + 3):                                                     # decode steps across a fold
        both(slice(r, r + 2))
        r += 2
    ip = torch.tensor([0, 3, 5], dtype=torch.int32)
    both(slice(r, r + 5), ip=ip, commit=False)                                 # verify: reads only
    both(slice(r, r + 5), ip=ip, commit=True)                                  # replay of the same rows
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert torch.equal(wg.win_len.cpu(), wc.win_len)
    live = slots.long()
    assert (wg.z[live.cuda()].cpu().int() - wc.z[live].int()).abs().max() <= 1        # rounding at .5 may differ
    assert torch.allclose(wg.zscale[live.cuda()].cpu(), wc.zscale[live], rtol=1e-3, atol=1e-6)
    dg, dc = ssm_window.to_dense(wg, dev(slots)).cpu(), ssm_window.to_dense(wc, slots)
    assert (dg - dc).abs().max() <= 2e-2 * dc.abs().max()
    ssm_window.from_dense(wg, dev(slots), dev(dc))
    ssm_window.from_dense(wc, slots, dc)
    assert (wg.z[live.cuda()].cpu().int() - wc.z[live].int()).abs().max() <= 1 and not wg.win_len.cpu()[live].any()


@pytest.mark.gpu
def test_engine_window_state_gpu():
    """Tiny hybrid MoE on the GPU with the int8w state: graphs == eager, speculation runs through the captured
    rounds (verify reads only, replay commits), tokens close to the fp32-state run."""
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import scaled, tiny_hybrid_moe
    t = scaled(tiny_hybrid_moe(), mamba_state=64)
    m = HybridModel(t, "cuda", seed=0, init_device="cpu")
    g = torch.Generator().manual_seed(0)
    pre = torch.randint(0, t.vocab, (40,), generator=g).tolist()
    prompts = [pre + torch.randint(0, t.vocab, (12,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=24)
    ref = [r.output_ids for r in Executor(m, max_batch=4, max_ctx=160, use_graphs=False).generate_batch(prompts, sp)]
    kw = dict(max_batch=4, max_ctx=160, state_dtype=torch.int8, state_window=8)
    eager = [r.output_ids for r in Executor(m, use_graphs=False, **kw).generate_batch(prompts, sp)]
    ex = Executor(m, use_graphs=True, **kw)
    ex.capture_graphs()
    got = [r.output_ids for r in ex.generate_batch(prompts, sp)]
    assert got == eager
    agree = sum(a == b for x_, y_ in zip(got, ref) for a, b in zip(x_, y_))
    assert [o[0] for o in got] == [o[0] for o in ref] and agree >= 0.5 * 72, agree
    spec = Executor(m, use_graphs=True, buckets=(1, 4), **kw)
    spec.enable_spec(2)
    spec.capture_graphs()
    out = [r.output_ids for r in spec.generate_batch(prompts, sp)]
    spec.state.check()
    assert all(len(o) == 24 for o in out) and spec.spec.graphs.rounds > 0
    agree = sum(a == b for x_, y_ in zip(out, ref) for a, b in zip(x_, y_))
    assert agree >= 0.4 * 72, agree
    torch.cuda.synchronize()
    assert nv.read_status() == 0


def _gdn_inputs(t, kh, vh, kd, seed=0):
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(t, kh * kd, generator=gen) * 0.5).bfloat16()
    k = (torch.randn(t, kh * kd, generator=gen) * 0.5).bfloat16()
    v = (torch.randn(t, vh * kd, generator=gen) * 0.5).bfloat16()
    g = -torch.rand(t, vh, generator=gen) * 0.2
    beta = torch.rand(t, vh, generator=gen)
    return q, k, v, g, beta


def test_delta_rule_over_window_records_cpu():
    kh, vh, kd, w = 2, 4, 16, 5
    q, k, v, g, beta = _gdn_inputs(30, kh, vh, kd)
    pool = _pool(vh, kh, kd, kd, w)
    ws = pool.window_state(0)
    ref = torch.zeros(7, vh, kd, kd)
    slot = torch.tensor([2], dtype=torch.int32)
    ys, yr = [], []
    for r in range(30):
        init = torch.tensor([0 if r == 0 else 1], dtype=torch.int32)
        sl = slice(r, r + 1)
        ys.append(ssm_window.step_delta(ws, q[sl], k[sl], v[sl], g[sl], beta[sl], slot, has_init=init))
        yr.append(recurrent.gdn_scan(q[sl], k[sl], v[sl], g[sl], beta[sl], ref, slot, slot, k_heads=kh, v_heads=vh,
                                     kdim=kd, vdim=kd, has_init=init))
    ys, yr = torch.cat(ys).float(), torch.cat(yr).float()
    assert (ys - yr).abs().max() <= 0.04 * yr.abs().max()
    dense = ssm_window.to_dense(ws, slot)[0]
    assert (dense - ref[2]).abs().max() <= 0.04 * ref[2].abs().max()
    # read-only rows equal the committing replay up to the fold the replay starts with
    q2, k2, v2, g2, b2 = _gdn_inputs(4, kh, vh, kd, seed=5)
    ip = torch.tensor([0, 4], dtype=torch.int32)
    before = ws.win_len.clone()
    ro = ssm_window.step_delta(ws, q2, k2, v2, g2, b2, slot, q_indptr=ip, commit=False)
    assert torch.equal(before, ws.win_len)
    co = ssm_window.step_delta(ws, q2, k2, v2, g2, b2, slot, q_indptr=ip)
    assert (ro.float() - co.float()).abs().max() <= 0.04 * ro.float().abs().max()


@pytest.mark.gpu
def test_delta_rule_window_kernel_and_engine_gpu():
    """The delta-rule mode of the kernel against its CPU reference (Flash-Next head geometry), and a Qwen3.8-hybrid
    style stack decoding with the int8w state through graphs and captured speculative rounds."""
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import qwen38_hybrid, scaled
    kh, vh, kd, w = 4, 12, 128, 8
    q, k, v, g, beta = _gdn_inputs(2 * (w + 6), kh, vh, kd, seed=2)
    cpu, gpu = _pool(vh, kh, kd, kd, w), _pool(vh, kh, kd, kd, w, "cuda")
    wc, wg = cpu.window_state(0), gpu.window_state(0)
    slots = torch.tensor([1, 3], dtype=torch.int32)
    r = 0
    for step in range(w + 4):
        sl = slice(r, r + 2)
        init = torch.tensor([0, 0] if step == 0 else [1, 1], dtype=torch.int32)
        yc = ssm_window.step_delta(wc, q[sl], k[sl], v[sl], g[sl], beta[sl], slots, has_init=init)
        yg = ssm_window.step_delta(wg, q[sl].cuda(), k[sl].cuda(), v[sl].cuda(), g[sl].cuda().contiguous(),
                                   beta[sl].cuda().contiguous(), slots.cuda(), has_init=init.cuda())
        assert (yg.float().cpu() - yc.float()).abs().max() <= 3e-2 * max(yc.float().abs().max().item(), 1e-3)
        r += 2
    ip = torch.tensor([0, 3, 4], dtype=torch.int32)
    sl = slice(r, r + 4)
    for commit in (False, True):
        yc = ssm_window.step_delta(wc, q[sl], k[sl], v[sl], g[sl], beta[sl], slots, q_indptr=ip, commit=commit)
        yg = ssm_window.step_delta(wg, q[sl].cuda(), k[sl].cuda(), v[sl].cuda(), g[sl].cuda().contiguous(),
                                   beta[sl].cuda().contiguous(), slots.cuda(), q_indptr=ip.cuda(), commit=commit)
        assert (yg.float().cpu() - yc.float()).abs().max() <= 3e-2 * max(yc.float().abs().max().item(), 1e-3)
    assert torch.equal(wg.win_len.cpu(), wc.win_len)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    t = scaled(qwen38_hybrid(), layers=4, hidden=512, vocab=2048, q_heads=4, kv_heads=2, head_dim=128, ffn=1024,
               gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=128, mtp_layers=1, mtp_depth=2, kv_dtype="bf16")
    m = HybridModel(t, "cuda", seed=0, init_device="cpu")
    gen = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, t.vocab, (n,), generator=gen).tolist() for n in (40, 27)]
    sp = SamplingParams(max_tokens=16)
    kw = dict(max_batch=2, max_ctx=128, state_dtype=torch.int8, state_window=8, radix_cache=False)
    eager = [r_.output_ids for r_ in Executor(m, use_graphs=False, **kw).generate_batch(prompts, sp)]
    ex = Executor(m, use_graphs=True, buckets=(1, 2), **kw)
    ex.capture_graphs()
    assert [r_.output_ids for r_ in ex.generate_batch(prompts, sp)] == eager
    spec = Executor(m, use_graphs=True, buckets=(1, 2), **kw)
    spec.enable_spec(2)
    spec.capture_graphs()
    out = [r_.output_ids for r_ in spec.generate_batch(prompts, sp)]
    assert all(len(o) == 16 for o in out) and spec.spec.graphs.rounds > 0
    torch.cuda.synchronize()
    assert nv.read_status() == 0
