"""conv1d / Mamba-2 scan / gated delta rule: chunk continuity on CPU, kernels vs fp32 references on GPU."""
import pytest
import torch

from hibana_b200.ops import recurrent as rec


def _mamba_inputs(t, heads, p, n, groups, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, heads * p, generator=g).bfloat16()
    bm = torch.randn(t, groups * n, generator=g).bfloat16()
    cm = torch.randn(t, groups * n, generator=g).bfloat16()
    dt = torch.randn(t, heads, generator=g).bfloat16()
    a_log = torch.rand(heads, generator=g) * 1.5
    dtb = torch.randn(heads, generator=g) * 0.5
    d = torch.randn(heads, generator=g)
    return x, bm, cm, dt, a_log, dtb, d


def test_mamba_chunked_equals_single_pass_cpu():
    heads, p, n, groups = 4, 32, 16, 1
    x, bm, cm, dt, a_log, dtb, d = _mamba_inputs(24, heads, p, n, groups)
    st = torch.zeros(3, heads, p, n)
    slot = torch.tensor([1], dtype=torch.int32)
    ip = lambda a, b: torch.tensor([a, b], dtype=torch.int32)
    kw = dict(heads=heads, groups=groups, head_dim=p, d_state=n)
    y = rec.mamba2_scan(x, bm, cm, dt, a_log, dtb, d, st, slot, slot, q_indptr=ip(0, 24),
                        has_init=torch.tensor([0], dtype=torch.int32), **kw)
    full_state = st[1].clone()
    st.zero_()
    y1 = rec.mamba2_scan(x[:10], bm[:10], cm[:10], dt[:10], a_log, dtb, d, st, slot, slot, q_indptr=ip(0, 10),
                         has_init=torch.tensor([0], dtype=torch.int32), **kw)
    y2 = rec.mamba2_scan(x[10:], bm[10:], cm[10:], dt[10:], a_log, dtb, d, st, slot, slot, q_indptr=ip(0, 14), **kw)
    assert torch.equal(torch.cat([y1, y2]), y) and torch.equal(st[1], full_state)


def test_conv_and_gdn_chunk_continuity_cpu():
    g = torch.Generator().manual_seed(1)
    c, w = 12, 4
    x = torch.randn(15, c, generator=g).bfloat16()
    wt = torch.randn(c, w, generator=g).bfloat16()
    st = torch.zeros(2, c, w - 1, dtype=torch.bfloat16)
    slot = torch.tensor([1], dtype=torch.int32)
    ip = lambda a, b: torch.tensor([a, b], dtype=torch.int32)
    zero = torch.tensor([0], dtype=torch.int32)
    y = rec.conv1d(x, wt, None, st, slot, slot, q_indptr=ip(0, 15), has_init=zero)
    st.zero_()
    y1 = rec.conv1d(x[:7], wt, None, st, slot, slot, q_indptr=ip(0, 7), has_init=zero)
    y2 = rec.conv1d(x[7:], wt, None, st, slot, slot, q_indptr=ip(0, 8))
    assert torch.equal(torch.cat([y1, y2]), y)
    kh, vh, kd, vd = 2, 4, 32, 32
    q = torch.randn(9, kh * kd, generator=g).bfloat16()
    k = torch.randn(9, kh * kd, generator=g).bfloat16()
    v = torch.randn(9, vh * vd, generator=g).bfloat16()
    gg = -torch.rand(9, vh, generator=g)
    beta = torch.rand(9, vh, generator=g)
    gs = torch.zeros(2, vh, vd, kd)
    kw = dict(k_heads=kh, v_heads=vh, kdim=kd, vdim=vd)
    o = rec.gdn_scan(q, k, v, gg, beta, gs, slot, slot, q_indptr=ip(0, 9), has_init=zero, **kw)
    gs.zero_()
    o1 = rec.gdn_scan(q[:4], k[:4], v[:4], gg[:4], beta[:4], gs, slot, slot, q_indptr=ip(0, 4), has_init=zero, **kw)
    o2 = rec.gdn_scan(q[4:], k[4:], v[4:], gg[4:].contiguous(), beta[4:].contiguous(), gs, slot, slot,
                      q_indptr=ip(0, 5), **kw)
    assert torch.equal(torch.cat([o1, o2]), o)


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item()), (a - b).abs().max().item()


@pytest.mark.gpu
@pytest.mark.parametrize("heads,p,n,groups", [(8, 32, 64, 1), (16, 64, 128, 8), (4, 64, 64, 2)])
def test_mamba_scan_gpu(heads, p, n, groups):
    rows = [5, 1, 17]
    t = sum(rows)
    x, bm, cm, dt, a_log, dtb, d = _mamba_inputs(t, heads, p, n, groups, seed=3)
    ip = torch.tensor([0, 5, 6, 23], dtype=torch.int32)
    st = torch.randn(6, heads, p, n) * 0.1
    sin = torch.tensor([1, 2, 3], dtype=torch.int32)
    sout = torch.tensor([4, 2, 5], dtype=torch.int32)
    init = torch.tensor([1, 1, 0], dtype=torch.int32)
    kw = dict(heads=heads, groups=groups, head_dim=p, d_state=n)
    st_c, st_g = st.clone(), st.clone().cuda()
    ref = rec.mamba2_scan(x, bm, cm, dt, a_log, dtb, d, st_c, sin, sout, q_indptr=ip, has_init=init, **kw)
    got = rec.mamba2_scan(x.cuda(), bm.cuda(), cm.cuda(), dt.cuda(), a_log.cuda(), dtb.cuda(), d.cuda(), st_g,
                          sin.cuda(), sout.cuda(), q_indptr=ip.cuda(), has_init=init.cuda(), **kw)
    _close(got, ref, 2e-2)
    _close(st_g, st_c, 1e-3)
    # verify (no state write) then replay of a prefix is bitwise equal to a direct run of that prefix
    st_v = st.clone().cuda()
    args = [a.cuda() for a in (x, bm, cm, dt, a_log, dtb, d)]
    full = rec.mamba2_scan(*args, st_v, sin.cuda(), None, q_indptr=ip.cuda(), has_init=init.cuda(), **kw)
    assert torch.equal(st_v.cpu(), st)
    assert torch.equal(full, got)


@pytest.mark.gpu
def test_conv1d_gpu():
    g = torch.Generator().manual_seed(2)
    c = 300
    x = torch.randn(40, c + 20, generator=g).bfloat16()[:, 10:10 + c]     # a column slice with a row pitch
    wt = torch.randn(c, 4, generator=g).bfloat16()
    bias = torch.randn(c, generator=g).bfloat16()
    ip = torch.tensor([0, 1, 30, 40], dtype=torch.int32)
    st = torch.randn(5, c, 3, generator=g).bfloat16()
    sin = torch.tensor([1, 2, 3], dtype=torch.int32)
    sout = torch.tensor([1, 4, 3], dtype=torch.int32)
    init = torch.tensor([1, 0, 1], dtype=torch.int32)
    st_c, st_g = st.clone(), st.clone().cuda()
    ref = rec.conv1d(x, wt, bias, st_c, sin, sout, q_indptr=ip, has_init=init)
    got = rec.conv1d(x.cuda(), wt.cuda(), bias.cuda(), st_g, sin.cuda(), sout.cuda(), q_indptr=ip.cuda(),
                     has_init=init.cuda())
    _close(got, ref, 2e-2)
    assert torch.equal(st_g.cpu(), st_c)


@pytest.mark.gpu
@pytest.mark.parametrize("kh,vh,kd", [(2, 4, 128), (4, 4, 64), (2, 6, 32)])
def test_gdn_scan_gpu(kh, vh, kd):
    g = torch.Generator().manual_seed(4)
    rows = [7, 1, 12]
    t = sum(rows)
    q = torch.randn(t, kh * kd, generator=g).bfloat16()
    k = torch.randn(t, kh * kd, generator=g).bfloat16()
    v = torch.randn(t, vh * kd, generator=g).bfloat16()
    gg = -torch.rand(t, vh, generator=g) * 0.5
    beta = torch.rand(t, vh, generator=g)
    ip = torch.tensor([0, 7, 8, 20], dtype=torch.int32)
    st = torch.randn(5, vh, kd, kd, generator=g) * 0.05
    sin = torch.tensor([1, 2, 3], dtype=torch.int32)
    sout = torch.tensor([1, 4, 3], dtype=torch.int32)
    init = torch.tensor([1, 0, 1], dtype=torch.int32)
    kw = dict(k_heads=kh, v_heads=vh, kdim=kd, vdim=kd)
    st_c, st_g = st.clone(), st.clone().cuda()
    ref = rec.gdn_scan(q, k, v, gg, beta, st_c, sin, sout, q_indptr=ip, has_init=init, **kw)
    got = rec.gdn_scan(q.cuda(), k.cuda(), v.cuda(), gg.cuda(), beta.cuda(), st_g, sin.cuda(), sout.cuda(),
                       q_indptr=ip.cuda(), has_init=init.cuda(), **kw)
    _close(got, ref, 3e-2)
    _close(st_g, st_c, 2e-3)


def _mamba_case(dtype, slots=5, heads=4, p=32, n=64, groups=1, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = 9
    x = torch.randn(t, heads * p, generator=g).bfloat16()
    bm = torch.randn(t, groups * n, generator=g).bfloat16()
    cm = torch.randn(t, groups * n, generator=g).bfloat16()
    dt = torch.randn(t, heads, generator=g).bfloat16()
    a_log = torch.randn(heads, generator=g) * 0.3
    state = torch.randn(slots, heads, p, n, generator=g) * 0.5
    scale = None
    if dtype == torch.int8:
        scale = state.abs().amax(-1) / 127
        state = torch.round(state / scale[..., None]).to(torch.int8)
    else:
        state = state.to(dtype)
    indptr = torch.tensor([0, 4, 9], dtype=torch.int32)
    slot_in = torch.tensor([1, 3], dtype=torch.int32)
    slot_out = torch.tensor([2, 3], dtype=torch.int32)
    return x, bm, cm, dt, a_log, state, scale, indptr, slot_in, slot_out, dict(heads=heads, groups=groups, head_dim=p, d_state=n)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.int8])
def test_mamba2_quantised_state_formats(dtype):
    """fp16 and int8 (+ row scale) pool representations: same recurrence, state requantised on write-back."""
    from hibana_b200.ops import recurrent
    x, bm, cm, dt, a_log, st, sc, ip, si, so, kw = _mamba_case(dtype)
    st_ref, sc_ref = st.clone(), sc.clone() if sc is not None else None
    y_ref = recurrent.mamba2_scan(x, bm, cm, dt, a_log, None, None, st_ref, si, so, q_indptr=ip, state_scale=sc_ref, **kw)
    st_g, sc_g = st.cuda(), sc.cuda() if sc is not None else None
    y = recurrent.mamba2_scan(x.cuda(), bm.cuda(), cm.cuda(), dt.cuda(), a_log.cuda(), None, None, st_g, si.cuda(),
                              so.cuda(), q_indptr=ip.cuda(), state_scale=sc_g, **kw)
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=3e-2, rtol=3e-2)
    deq = lambda s, c: s.float() * (c[..., None] if c is not None else 1.0)  # noqa: E731
    a, b = deq(st_g.cpu(), sc_g.cpu() if sc_g is not None else None), deq(st_ref, sc_ref)
    tol = 2e-2 if dtype == torch.float16 else 4e-2
    assert float((a[[2, 3]] - b[[2, 3]]).abs().max()) < tol * float(b[[2, 3]].abs().max())
    assert torch.equal(a[[0, 1, 4]], b[[0, 1, 4]])          # untouched slots


@pytest.mark.gpu
def test_fp16_stochastic_rounding_is_unbiased():
    """A state of 1.0 decayed by 1 - 0.3 * 2^-11 lies between two fp16 neighbours: round-to-nearest stores 1.0 every
    time (the decay is lost for ever), stochastic rounding stores the right value on average."""
    import math
    from hibana_b200.ops import recurrent
    heads, p, n = 4, 32, 64
    raw = torch.tensor([[-8.8125] * heads]).bfloat16()
    dtv = math.log1p(math.exp(float(raw[0, 0])))
    decay = math.exp(-dtv)                                   # a = -exp(0) = -1
    frac = (1.0 - decay) / 2 ** -11
    assert 0.2 < frac < 0.45
    x = torch.zeros(1, heads * p).bfloat16().cuda()
    bm = torch.zeros(1, n).bfloat16().cuda()
    a_log = torch.zeros(heads).cuda()
    si, so = torch.tensor([1], dtype=torch.int32).cuda(), torch.tensor([2], dtype=torch.int32).cuda()
    kw = dict(heads=heads, groups=1, head_dim=p, d_state=n)
    st = torch.zeros(3, heads, p, n, dtype=torch.float16, device="cuda")
    st[1] = 1.0
    recurrent.mamba2_scan(x, bm, bm, raw.cuda(), a_log, None, None, st, si, so, sr_seed=0, **kw)
    assert float(st[2].float().mean()) == 1.0
    recurrent.mamba2_scan(x, bm, bm, raw.cuda(), a_log, None, None, st, si, so, sr_seed=1234, **kw)
    vals = st[2].float()
    assert set(vals.unique().tolist()) <= {1.0, 1.0 - 2 ** -11}
    err = abs(float(vals.double().mean()) - decay)
    assert err < 0.03 * 2 ** -11, (err / 2 ** -11, frac)
