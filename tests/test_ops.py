"""Row / attention / sampling kernels against the plain-PyTorch references (which run on CPU)."""
import math

import pytest
import torch

from hibana_b200.ops import attention, basic, nvfp4, sampling


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item()), (a - b).abs().max().item()


@pytest.mark.gpu
@pytest.mark.parametrize("h", [256, 2560, 5120, 8192])
@pytest.mark.parametrize("gemma", [False, True])
def test_rmsnorm(h, gemma):
    x = torch.randn(37, h).bfloat16()
    r = torch.randn(37, h).bfloat16()
    w = (torch.randn(h) * 0.1).bfloat16()
    rc, rg = r.clone(), r.clone().cuda()
    ref = basic.rmsnorm(x, w, 1e-6, residual=rc, gemma=gemma)
    got = basic.rmsnorm(x.cuda(), w.cuda(), 1e-6, residual=rg, gemma=gemma)
    _close(got, ref, 2e-2)
    assert torch.equal(rg.cpu(), rc)
    _close(basic.rmsnorm(x.cuda(), w.cuda(), 1e-6), basic.rmsnorm(x, w, 1e-6), 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("norm_first,sig", [(False, False), (True, False), (True, True)])
def test_gated_rmsnorm(norm_first, sig):
    x, z = torch.randn(19, 1024).bfloat16(), torch.randn(19, 1024).bfloat16()
    w = torch.randn(1024).bfloat16()
    ref = basic.gated_rmsnorm(x, z, w, 1e-5, 128, norm_first=norm_first, sigmoid_gate=sig)
    got = basic.gated_rmsnorm(x.cuda(), z.cuda(), w.cuda(), 1e-5, 128, norm_first=norm_first, sigmoid_gate=sig)
    _close(got, ref, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("d,rot,qk_norm,fp8,q_gate", [(128, 128, False, False, False), (256, 64, True, True, True),
                                                      (64, 64, False, False, False), (128, 0, False, False, False)])
def test_rope_kv_write(d, rot, qk_norm, fp8, q_gate):
    hq, hkv, t = 6, 2, 23
    width = hq * d * (2 if q_gate else 1) + 2 * hkv * d
    qkv = torch.randn(t, width).bfloat16()
    pos = torch.randint(0, 100000, (t,), dtype=torch.int32)
    slots = torch.randperm(64)[:t].int() + 1
    inv = basic.rope_inv_freq(max(rot, 2), 1e6)
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    qn = (torch.randn(d) * 0.1).bfloat16() if qk_norm else None
    kn = (torch.randn(d) * 0.1).bfloat16() if qk_norm else None
    outs = []
    for dev in ("cpu", "cuda"):
        kp = torch.zeros(80, hkv, d, dtype=dt, device=dev)
        vp = torch.zeros(80, hkv, d, dtype=dt, device=dev)
        q = basic.rope_kv_write(qkv.to(dev), pos.to(dev), slots.to(dev), inv.to(dev), kp, vp, hq, hkv, d, rot=rot,
                                q_norm=None if qn is None else qn.to(dev), k_norm=None if kn is None else kn.to(dev),
                                gemma_norm=qk_norm, kv_scale=0.5 if fp8 else 1.0, q_gate=q_gate)
        outs.append((q, kp, vp))
    _close(outs[1][0], outs[0][0], 3e-2)
    _close(outs[1][1].float(), outs[0][1].float(), 7e-2 if fp8 else 3e-2)
    _close(outs[1][2].float(), outs[0][2].float(), 7e-2 if fp8 else 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("d,q_gate", [(64, False), (128, False), (256, True)])
def test_rope_kv_write_with_angle_table(d, q_gate):
    """Prefill-sized calls take the angles from a per-forward table; the plain case (bf16 pools, full rotary, no
    q / k norm) runs the vectorised kernel, anything else the generic one with the same table. Both equal the
    table-free kernel up to the rounding of a fused multiply-add and the CPU reference within tolerance."""
    from types import SimpleNamespace
    hq, hkv, t = 6, 2, 300
    width = hq * d * (2 if q_gate else 1) + 2 * hkv * d
    qkv = torch.randn(t, width).bfloat16().cuda()
    pos = torch.randint(0, 100000, (t,), dtype=torch.int32).cuda()
    slots = (torch.randperm(400)[:t].int() + 1).cuda()
    inv = basic.rope_inv_freq(d, 1e6).cuda()
    ctx = SimpleNamespace(positions=pos, extras={})
    table = basic.rope_table(ctx, inv, d)
    assert table is not None and table.shape == (t, d // 2, 2) and basic.rope_table(ctx, inv, d) is table
    assert basic.rope_table(SimpleNamespace(positions=pos[:8], extras={}), inv, d) is None      # decode-sized: no table
    for norm in (False, True):
        qn = (torch.randn(d) * 0.1).bfloat16().cuda() if norm else None
        got, want = [], []
        for tab, outs in ((table, got), (None, want)):
            kp = torch.zeros(420, hkv, d, dtype=torch.bfloat16, device="cuda")
            vp = torch.zeros(420, hkv, d, dtype=torch.bfloat16, device="cuda")
            q = basic.rope_kv_write(qkv, pos, slots, inv, kp, vp, hq, hkv, d, q_norm=qn, k_norm=qn, q_gate=q_gate,
                                    table=tab)
            outs.extend((q, kp, vp))
        for a, b in zip(got, want):          # same angles; products may contract differently: one bf16 step at most
            _close(a.float(), b.float(), 1e-2)
            assert (a.float() != b.float()).float().mean() < 0.02
    kp = torch.zeros(420, hkv, d, dtype=torch.bfloat16)
    vp = torch.zeros(420, hkv, d, dtype=torch.bfloat16)
    q = basic.rope_kv_write(qkv.cpu(), pos.cpu(), slots.cpu(), inv.cpu(), kp, vp, hq, hkv, d, q_gate=q_gate)
    kp2 = torch.zeros(420, hkv, d, dtype=torch.bfloat16, device="cuda")
    vp2 = torch.zeros(420, hkv, d, dtype=torch.bfloat16, device="cuda")
    q2 = basic.rope_kv_write(qkv, pos, slots, inv, kp2, vp2, hq, hkv, d, q_gate=q_gate, table=table)
    _close(q2, q, 3e-2)
    _close(kp2.float(), kp.float(), 3e-2)
    _close(vp2.float(), vp.float(), 3e-2)


@pytest.mark.gpu
def test_act_embedding_add():
    x = torch.randn(33, 512).bfloat16()
    for mode in (basic.ACT_SILU_SPLIT, basic.ACT_SILU_PAIRS, basic.ACT_RELU2):
        _close(basic.act_mul(x.cuda(), mode), basic.act_mul(x, mode), 2e-2)
    g = torch.randn(33, 512).bfloat16()
    _close(basic.act_mul(x.cuda(), basic.ACT_SIGMOID_GATE, g.cuda()), basic.act_mul(x, basic.ACT_SIGMOID_GATE, g), 2e-2)
    table = torch.randn(100, 256).bfloat16()
    ids = torch.randint(0, 100, (17,))
    assert torch.equal(basic.embedding(ids.cuda(), table.cuda()).cpu(), basic.embedding(ids, table))
    _close(basic.add(x.cuda(), g.cuda()), basic.add(x, g), 1e-2)


def _attn_case(b, rows, ctxs, hq, hkv, d, dtype=torch.bfloat16, seed=0, contiguous=False):
    g = torch.Generator().manual_seed(seed)
    total = sum(ctxs)
    slots_n = total + 8
    kp = (torch.randn(slots_n, hkv, d, generator=g) * 0.7)
    vp = torch.randn(slots_n, hkv, d, generator=g)
    perm = torch.randperm(slots_n - 1, generator=g) + 1
    if contiguous:      # ascending runs, as a fresh pool hands them out (bulk-copy path), with one hole
        perm = torch.arange(1, slots_n)
        perm[40], perm[41] = perm[41].clone(), perm[40].clone()
    kv_idx = torch.zeros(b + 2, max(ctxs) + 3, dtype=torch.int32)
    seq_rows = torch.arange(b, dtype=torch.int32).flip(0) + 1   # non-identity rows
    o = 0
    for i, c in enumerate(ctxs):
        kv_idx[seq_rows[i], :c] = perm[o:o + c].int()
        o += c
    q = torch.randn(sum(rows), hq, d, generator=g).bfloat16()
    indptr = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    ctx = torch.tensor(ctxs, dtype=torch.int32)
    if dtype == torch.bfloat16:
        kp, vp = kp.bfloat16(), vp.bfloat16()
    else:
        kp, vp = (kp / 0.25).to(dtype), (vp / 0.25).to(dtype)
    if contiguous is True:      # head-major storage behind the [slots, heads, D] view, as the engine's pool
        kp = kp.transpose(0, 1).contiguous().transpose(0, 1)
        vp = vp.transpose(0, 1).contiguous().transpose(0, 1)
    return q, kp, vp, kv_idx, ctx, indptr, seq_rows


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,d", [(40, 8, 128), (4, 2, 64), (24, 2, 256), (32, 2, 128)])
@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("contiguous", [False, True])
def test_paged_attention_decode(hq, hkv, d, splits, contiguous):
    ctxs = [1, 63, 64, 65, 300, 1000]
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(6, [1] * 6, ctxs, hq, hkv, d, contiguous=contiguous)
    ref = attention.paged_attention(q, kp, vp, idx, ctx, seq_rows=sr)
    got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(), seq_rows=sr.cuda(),
                                    splits=splits)
    _close(got, ref, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_paged_attention_ragged_rows(fp8):
    rows, ctxs = [4, 1, 16, 33, 7], [10, 200, 16, 150, 500]
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(5, rows, ctxs, 10, 2, 128, dtype=dt)
    scale = 0.25 if fp8 else 1.0
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=33, seq_rows=sr, kv_scale=scale)
    for splits in (1, 3):
        got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(),
                                        q_indptr=indptr.cuda(), max_rows=33, seq_rows=sr.cuda(), kv_scale=scale,
                                        splits=splits)
        _close(got, ref, 3e-2)


@pytest.mark.gpu
def test_argmax_and_sampling():
    logits = torch.randn(9, 5000)
    logits[3, 77] = logits[3, 4000] = 50.0          # exact tie -> lowest index
    assert sampling.argmax(logits.cuda()).cpu().tolist() == sampling.argmax(logits).tolist()
    assert sampling.argmax(logits.cuda())[3].item() == 77
    bits = torch.zeros(9, (5000 + 31) // 32, dtype=torch.int32)
    allowed = torch.randint(0, 5000, (9, 40))
    for r in range(9):
        for a in allowed[r].tolist():
            bits[r, a // 32] |= (1 << (a % 32)) if a % 32 != 31 else -(1 << 31)
    assert sampling.argmax(logits.cuda(), bits.cuda()).cpu().tolist() == sampling.argmax(logits, bits).tolist()
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.0, 1.0, 1.0, 2.0, 0.5])
    top_k = torch.tensor([0, 5, 64, 0, 1, 1, 20, 50, 3], dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5, 1.0, 1.0, 0.8, 1.0, 0.99])
    seeds = torch.arange(9, dtype=torch.int64) * 7919 + 13
    offs = torch.arange(9, dtype=torch.int64)
    ref = sampling.sample(logits, temp, top_k, top_p, seeds, offs)
    got = sampling.sample(logits.cuda(), temp.cuda(), top_k.cuda(), top_p.cuda(), seeds.cuda(), offs.cuda())
    assert got.cpu().tolist() == ref.tolist()


def test_sampling_distribution_cpu():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4000, 1)
    n = 4000
    out = sampling.sample(logits, torch.ones(n), torch.zeros(n, dtype=torch.int32), torch.ones(n),
                          torch.full((n,), 5, dtype=torch.int64), torch.arange(n, dtype=torch.int64))
    freq = torch.bincount(out, minlength=4).float() / n
    assert (freq - torch.softmax(logits[0], 0)).abs().max() < 0.03


def test_accept_greedy_cpu_and_rank_gap():
    target = torch.tensor([[5, 6, 7, 8], [5, 6, 7, 8], [1, 2, 3, 4], [9, 9, 9, 9]])
    drafts = torch.tensor([[5, 6, 7], [5, 0, 7], [0, 2, 3], [9, 9, 9]])
    e, c, a = sampling.accept_greedy(target, drafts)
    assert c.tolist() == [4, 2, 1, 4] and a.tolist() == [3, 1, 0, 3]
    assert e[1, :2].tolist() == [5, 6]
    e, c, a = sampling.accept_greedy(target, drafts, stop_ids=torch.tensor([[6], [6], [6], [6]]))
    assert c.tolist() == [2, 2, 1, 4]
    e, c, a = sampling.accept_greedy(target, drafts, budget=torch.tensor([2, 9, 9, 3], dtype=torch.int32))
    assert c.tolist() == [2, 2, 1, 3]
    lg = torch.tensor([[1.0, 3.0, 2.0, 0.5]])
    r, g = sampling.rank_gap(lg, torch.tensor([2]))
    assert r.tolist() == [1] and abs(g.item() - 1.0) < 1e-6


@pytest.mark.gpu
def test_accept_greedy_and_rank_gap_gpu():
    g = torch.Generator().manual_seed(3)
    target = torch.randint(0, 4, (64, 6), generator=g)
    drafts = torch.randint(0, 4, (64, 5), generator=g)
    stops = torch.randint(0, 8, (64, 2), generator=g)
    budget = torch.randint(1, 7, (64,), generator=g, dtype=torch.int32)
    depth = torch.randint(0, 6, (64,), generator=g, dtype=torch.int32)
    ref = sampling.accept_greedy(target, drafts, stops, budget, depth)
    got = sampling.accept_greedy(target.cuda(), drafts.cuda(), stops.cuda(), budget.cuda(), depth.cuda())
    assert got[1].cpu().tolist() == ref[1].tolist() and got[2].cpu().tolist() == ref[2].tolist()
    for i in range(64):
        n = int(ref[1][i])
        assert got[0][i, :n].cpu().tolist() == ref[0][i, :n].tolist()
    lg = torch.randn(11, 3000)
    ids = torch.randint(0, 3000, (11,))
    r1, g1 = sampling.rank_gap(lg, ids)
    r2, g2 = sampling.rank_gap(lg.cuda(), ids.cuda())
    assert r1.tolist() == r2.cpu().tolist() and torch.allclose(g1, g2.cpu(), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,d,rows", [(40, 8, 128, [3, 1, 2, 3]), (4, 2, 64, [8, 1, 5, 2]), (12, 2, 256, [2, 1, 2, 1])])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("contiguous", [False, True, "slot-major"])
def test_tensor_core_decode_verify_rows(hq, hkv, d, rows, splits, contiguous):
    ctxs = [40, 700, 129, 2500]
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(4, rows, ctxs, hq, hkv, d, seed=5, contiguous=contiguous)
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=max(rows), seq_rows=sr)
    got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(), q_indptr=indptr.cuda(),
                                    max_rows=max(rows), seq_rows=sr.cuda(), splits=splits)
    _close(got, ref, 2e-2)
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,rows", [(40, 8, [3, 1, 2, 3]), (16, 2, [2, 1, 1, 2]), (8, 8, [1, 1, 1, 1])])
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("contiguous", [False, True, "slot-major"])
def test_tcgen05_decode_kernel(hq, hkv, rows, splits, contiguous):
    """The persistent tcgen05 decode kernel (opt-in): ragged contexts, empty splits, multi-row verify, all layouts."""
    from hibana_b200 import config as cfgmod
    ctxs = [40, 700, 129, 2500]
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(4, rows, ctxs, hq, hkv, 128, seed=7, contiguous=contiguous)
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=max(rows), seq_rows=sr)
    with cfgmod.using(decode_attn="tc"):
        got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(),
                                        q_indptr=indptr.cuda(), max_rows=max(rows), seq_rows=sr.cuda(), splits=splits)
    _close(got, ref, 2e-2)
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,d", [(40, 8, 128), (4, 2, 64), (32, 2, 128), (3, 1, 64), (24, 2, 256), (4, 4, 256)])
@pytest.mark.parametrize("contiguous", [False, True, "slot-major"])
def test_tcgen05_prefill_attention(hq, hkv, d, contiguous):
    """Ragged prefill / chunked prefill over cached prefixes: tile edges, partial query blocks, 1-row sequences."""
    rows, ctxs = [300, 17, 128, 1, 257], [300, 500, 1200, 77, 257]
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(5, rows, ctxs, hq, hkv, d, seed=11, contiguous=contiguous)
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=max(rows), seq_rows=sr)
    got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(), q_indptr=indptr.cuda(),
                                    max_rows=max(rows), seq_rows=sr.cuda())
    _close(got, ref, 2e-2)
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0
    # non-causal (encoder-style) rows see the whole context
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=max(rows), seq_rows=sr,
                                    causal=False)
    got = attention.paged_attention(q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda(), q_indptr=indptr.cuda(),
                                    max_rows=max(rows), seq_rows=sr.cuda(), causal=False)
    _close(got, ref, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,d,rows", [(40, 8, 128, [1, 1, 1, 1]), (40, 8, 128, [3, 1, 2, 3]), (4, 2, 64, [2, 1, 1, 2])])
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("in_kernel", [True, False])
def test_decode_attention_fused_merge_and_quant(hq, hkv, d, rows, splits, in_kernel):
    """In-kernel split merge (last-arriving CTA) and NVFP4 output of the decode kernel: the merged rows match the
    separate merge kernel's, the NVFP4 rows equal quantising the kernel's bf16 rows afterwards byte for byte, twice in a row
    (the arrival counters re-arm themselves), and both stay close to the fp32 reference."""
    from hibana_b200 import _native as nv
    from hibana_b200 import config as cfgmod
    from hibana_b200.ops import nvfp4
    ctxs = [40, 700, 129, 2500]
    q, kp, vp, idx, ctx, indptr, sr = _attn_case(4, rows, ctxs, hq, hkv, d, seed=11, contiguous=True)
    ref = attention.paged_attention(q, kp, vp, idx, ctx, q_indptr=indptr, max_rows=max(rows), seq_rows=sr)
    args = (q.cuda(), kp.cuda(), vp.cuda(), idx.cuda(), ctx.cuda())
    kw = dict(q_indptr=indptr.cuda(), max_rows=max(rows), seq_rows=sr.cuda(), splits=splits)
    with cfgmod.using(fuse_epilogues=False):
        plain = attention.paged_attention(*args, **kw)
    gs = torch.tensor(2.0 / (6 * 448), device="cuda")
    ws = attention.AttnWorkspace(q.shape[0], hq, d, splits, torch.device("cuda")) if splits > 1 else None
    for _ in range(2):
        # in_kernel: the last-arriving split CTA merges and quantises; else the merge kernel writes the NVFP4 rows
        with cfgmod.using(fuse_attn_tail=in_kernel):
            fused = attention.paged_attention(*args, workspace=ws, **kw)
            _close(fused, plain, 8e-3)          # same sums, possibly contracted differently
            want = nvfp4.quantize(fused.view(fused.shape[0], -1), gs)
            xq = attention.paged_attention(*args, workspace=ws, quant_scale=gs, **kw)
        assert torch.equal(xq.q, want.q)
        groups = hq * d // 16
        assert torch.equal(nvfp4.unswizzle_sf(xq.sf, xq.rows, groups), nvfp4.unswizzle_sf(want.sf, want.rows, groups))
    _close(plain, ref, 2e-2)
    assert nv.read_status() == 0


def test_sampling_full_vocab_law_cpu():
    """top_k = 0 samples the whole vocabulary: the empirical law matches `distribution`, also under top-p."""
    from hibana_b200.engine.rejection import distribution
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5] + [-3.0] * 95]).repeat(3000, 1)
    n = 3000
    for p in (1.0, 0.8):
        out = sampling.sample(logits, torch.ones(n), torch.zeros(n, dtype=torch.int32), torch.full((n,), p),
                              torch.full((n,), 11, dtype=torch.int64), torch.arange(n, dtype=torch.int64))
        freq = torch.bincount(out, minlength=100).float() / n
        law = distribution(logits[:1], 1.0, 0, p)[0]
        assert (freq - law).abs().max() < 0.03
        assert freq[law == 0].sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.3])
def test_sampling_full_vocab_kernel_matches_distribution(top_p):
    """Kernel path for top_k = 0 / > 64: every draw lands inside the law's support, the reported probability of
    the drawn token equals the law's, the empirical frequencies follow it, and ties at the nucleus edge are cut in
    index order."""
    from hibana_b200.engine.rejection import distribution
    g = torch.Generator().manual_seed(3)
    vocab, n = 3000, 4096
    row = torch.randn(vocab, generator=g) * 2.0
    row[100:110] = row[5]                  # ties
    logits = row[None, :].repeat(n, 1).cuda()
    temp = torch.full((n,), 0.8, device="cuda")
    top_k = torch.zeros(n, dtype=torch.int32, device="cuda")
    top_k[::2] = 100                        # > 64 takes the same path
    tp = torch.full((n,), top_p, device="cuda")
    seeds = torch.full((n,), 77, dtype=torch.int64, device="cuda")
    offs = torch.arange(n, dtype=torch.int64, device="cuda")
    out = sampling.sample(logits, temp, top_k, tp, seeds, offs)
    picks = out.cpu()
    for start, k in ((1, 0), (0, 100)):      # odd rows: whole vocabulary; even rows: exactly the 100 largest
        law = distribution(row[None, :], 0.8, k, top_p)[0]
        mine = picks[start::2]
        assert (law[mine] > 0).all()
        freq = torch.bincount(mine, minlength=vocab).float() / mine.numel()
        assert (freq - law).abs().max() < 0.04
    # the CPU statement of the same rule makes the same draws, up to rounding at CDF edges
    ref = sampling.sample(logits.cpu(), temp.cpu(), top_k.cpu(), tp.cpu(), seeds.cpu(), offs.cpu())
    assert (ref == picks).float().mean() > 0.99


def _spec_case(dev, b=24, k=3, vocab=2000, seed=5):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(b * (k + 1), vocab, generator=g) * 3.0
    logits[:, 40:48] = logits[:, 7:8]                       # ties around likely thresholds
    top = logits.view(b, k + 1, vocab)[:, :k].argmax(-1)
    drafts = torch.where(torch.rand(b, k, generator=g) < 0.6, top, torch.randint(0, vocab, (b, k), generator=g))
    temp = torch.tensor([0.0 if i % 6 == 0 else 0.7 + 0.1 * (i % 4) for i in range(b)])
    top_k = torch.tensor([(0, 20, 100, 5)[i % 4] for i in range(b)], dtype=torch.int32)
    top_p = torch.tensor([(1.0, 0.9, 0.5)[i % 3] for i in range(b)])
    seeds = torch.arange(b, dtype=torch.int64) + 1000
    draws = torch.arange(b, dtype=torch.int64) * 3
    soft = torch.tensor([0.5 if i % 5 == 0 else 0.0 for i in range(b)])
    return [x.to(dev) for x in (logits, drafts, temp, top_k, top_p, seeds, draws, soft)]


def test_spec_targets_reference_is_rejection_sampling_cpu():
    """The targets rule + exact-prefix accept equals `verify_batch` with point-mass draft laws on the same uniforms."""
    from hibana_b200.engine import rejection
    logits, drafts, temp, top_k, top_p, seeds, draws, soft = _spec_case("cpu")
    soft = torch.zeros_like(soft)
    b, k = drafts.shape
    target, p_draft = sampling.spec_targets(logits, drafts, temp, top_k, top_p, seeds, draws, soft)
    emitted, count, accepted = sampling.accept_greedy(target, drafts)
    laws = rejection.distribution(logits, temp.repeat_interleave(k + 1), top_k.repeat_interleave(k + 1),
                                  top_p.repeat_interleave(k + 1)).view(b, k + 1, -1)
    q = torch.zeros(b, k, logits.shape[1]).scatter_(2, drafts[:, :, None], 1.0)
    u = torch.tensor([[[sampling.uniform01(int(seeds[i]), 2 * (int(draws[i]) + j) + 1 + t) for t in range(2)]
                       for j in range(k + 1)] for i in range(b)])
    ver = rejection.verify_batch(laws, q, drafts, u[..., 0].contiguous(), u[..., 1].contiguous())
    assert torch.equal(accepted, ver.accepted) and torch.equal(count, ver.count)
    for i in range(b):
        assert torch.equal(emitted[i, :int(count[i])], ver.emitted[i, :int(count[i])]), i
    assert torch.allclose(p_draft[:, :k], laws[:, :k].gather(2, drafts[:, :, None]).squeeze(2), atol=1e-6)


@pytest.mark.gpu
def test_spec_targets_kernel_matches_reference():
    """One kernel for sampled verification: same law (temperature, top-k with ties, nucleus), same uniforms, same
    accepted drafts and correction / bonus draws as the PyTorch statement; greedy and relaxed requests included."""
    args = _spec_case("cuda")
    target, p_draft = sampling.spec_targets(*args)
    ref_t, ref_p = sampling.spec_targets(*[a.cpu() for a in args])
    assert torch.allclose(p_draft.cpu(), ref_p, atol=2e-4, rtol=1e-3)
    same = (target.cpu() == ref_t)
    assert same.float().mean() > 0.97, same.float().mean()       # rounding at CDF edges may move a draw
    drafts = args[1]
    stands = target[:, :-1] == drafts
    assert torch.equal(stands.cpu(), ref_t[:, :-1] == drafts.cpu()) or same.float().mean() > 0.99
    greedy = (args[2] <= 0).cpu()
    lg = args[0].view(drafts.shape[0], drafts.shape[1] + 1, -1)
    assert torch.equal(target.cpu()[greedy], lg.argmax(-1).cpu()[greedy])      # temperature 0: the argmax, every row
    # bf16 logits take the same path
    t16, _ = sampling.spec_targets(args[0].bfloat16(), *args[1:])
    r16, _ = sampling.spec_targets(args[0].bfloat16().cpu(), *[a.cpu() for a in args[1:]])
    assert (t16.cpu() == r16).float().mean() > 0.97
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("gs,h,norm_first", [(1024, 4096, False), (128, 1536, True), (512, 1024, False)])
def test_gated_rmsnorm_quant_equals_norm_then_quantise(gs, h, norm_first):
    g = torch.Generator().manual_seed(1)
    rows = 19
    x = torch.randn(rows, h + 64, generator=g).bfloat16().cuda()[:, :h]          # strided rows
    z = torch.randn(rows, h, generator=g).bfloat16().cuda()
    w = (torch.randn(h, generator=g) * 0.1 + 1).bfloat16().cuda()
    scale = torch.tensor([4.0 / (6 * 448)], device="cuda")
    ref = basic.gated_rmsnorm(x, z, w, 1e-5, gs, norm_first=norm_first)
    cpu = basic.gated_rmsnorm(x.cpu(), z.cpu(), w.cpu(), 1e-5, gs, norm_first=norm_first)
    _close(ref.cpu(), cpu, 2e-2)
    want = nvfp4.quantize(ref, scale)
    got = basic.gated_rmsnorm_quant(x, z, w, 1e-5, gs, scale, norm_first=norm_first)
    assert torch.equal(got.q, want.q)
    groups = h // 16
    assert torch.equal(nvfp4.unswizzle_sf(got.sf, rows, groups), nvfp4.unswizzle_sf(want.sf, rows, groups))


@pytest.mark.gpu
def test_gdn_gates_kernel():
    g = torch.Generator().manual_seed(2)
    ba = (torch.randn(33, 96, generator=g) * 3).bfloat16()
    a_log, dtb = torch.randn(48, generator=g), torch.randn(48, generator=g)
    beta, gg = basic.gdn_gates(ba, a_log, dtb)
    b2, g2 = basic.gdn_gates(ba.cuda(), a_log.cuda(), dtb.cuda())
    assert torch.allclose(b2.cpu(), beta, atol=1e-5) and torch.allclose(g2.cpu(), gg, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_lattice_walk_kernel_matches_torch():
    g = torch.Generator().manual_seed(4)
    b, k, w = 37, 5, 12
    cand = torch.randint(0, 3000, (b, k, w), generator=g)
    scores = torch.randn(b, k, w, w, generator=g) * 2
    scores[3, 1, :, 2] = scores[3, 1, :, 5] = 9.0                 # tie: the lower candidate index wins
    temp = torch.tensor([0.0 if i % 4 == 0 else 0.6 + 0.05 * i for i in range(b)])
    u = torch.rand(b, k, generator=g)
    for args in ((None, None), (temp, u)):
        ref = sampling.lattice_walk(cand, scores, *args)
        got = sampling.lattice_walk(cand.cuda(), scores.cuda(), *[a.cuda() if a is not None else None for a in args])
        same = (got[0].cpu() == ref[0]).float().mean()
        assert same == 1.0 if args[0] is None else same > 0.97
        if args[0] is None:
            assert torch.equal(got[1].cpu(), ref[1])
            assert torch.allclose(got[2].cpu(), ref[2], atol=1e-5) and torch.allclose(got[3].cpu(), ref[3], atol=1e-5)
    assert int(sampling.lattice_walk(cand.cuda(), scores.cuda())[1][3, 1]) == 2


def _fp4_case(dev, hq=8, hkv=2, d=128, t=70, seed=3):
    from hibana_b200.cache.kv_pool import KvPool
    g = torch.Generator().manual_seed(seed)
    pool = KvPool(1, 96, hkv, d, "nvfp4", dev)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, generator=g) * 1.5).bfloat16().to(dev)
    pos = torch.arange(t, dtype=torch.int32, device=dev)
    slots = (torch.randperm(95, generator=g)[:t].int() + 1).to(dev)
    inv = basic.rope_inv_freq(d, 1e6).to(dev)
    q = basic.rope_kv_write(qkv, pos, slots, inv, pool.k[0], pool.v[0], hq, hkv, d, kv_scale=pool.kv_scale)
    return pool, q, slots, qkv


def test_nvfp4_kv_pool_write_and_attention_cpu():
    """NVFP4 KV: rows are quantised on write (4.5 bits per element), attention over the pool equals fp32 attention
    over the dequantised rows, and the rows stay within NVFP4 rounding of what was written."""
    from hibana_b200.cache.kv_pool import KvPool
    pool, q, slots, qkv = _fp4_case("cpu")
    assert pool.bytes_per_token == 2 * 2 * (64 + 8) and pool.k[0].dtype == torch.uint8
    kd = pool.dequantized(0, 0, slots.tolist())
    bf = KvPool(1, 96, 2, 128, torch.bfloat16, "cpu")
    basic.rope_kv_write(qkv, torch.arange(70, dtype=torch.int32), slots, basic.rope_inv_freq(128, 1e6), bf.k[0],
                        bf.v[0], 8, 2, 128)
    want = bf.k[0][slots.long()].float()
    assert float((kd - want).norm() / want.norm()) < 0.12
    idx = slots.view(1, -1)
    ctx = torch.tensor([70], dtype=torch.int32)
    out = attention.paged_attention(q[-1:], pool.k[0], pool.v[0], idx, ctx, kv_scale=pool.kv_scale)
    k, v = pool.dequantized(0, 0, slots.tolist()), pool.dequantized(0, 1, slots.tolist())
    qq = q[-1].float().view(2, 4, 128)
    s = torch.einsum("hgd,chd->hgc", qq, k) / 128 ** 0.5
    ref = torch.einsum("hgc,chd->hgd", torch.softmax(s, -1), v).reshape(1, 8, 128)
    _close(out, ref, 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 3])
def test_nvfp4_kv_kernels_match_reference(rows):
    """GPU: the write kernel produces the reference quantiser's bytes, and the attention kernel over the NVFP4
    pool matches the CPU reference over the same pool (decode and a short verify block, split and unsplit)."""
    cpu, qc, slots, _ = _fp4_case("cpu")
    gpu, qg, _, _ = _fp4_case("cuda")
    sl = slots.long()
    assert torch.equal(gpu.k[0][sl.cuda()].cpu(), cpu.k[0][sl]) and torch.equal(gpu.k[0].sf[sl.cuda()].cpu(), cpu.k[0].sf[sl])
    assert torch.equal(gpu.v[0][sl.cuda()].cpu(), cpu.v[0][sl]) and torch.equal(gpu.v[0].sf[sl.cuda()].cpu(), cpu.v[0].sf[sl])
    _close(qg, qc, 2e-2)
    idx = slots.view(1, -1)
    ctx = torch.tensor([70], dtype=torch.int32)
    indptr = torch.tensor([0, rows], dtype=torch.int32)
    ref = attention.paged_attention(qc[-rows:], cpu.k[0], cpu.v[0], idx, ctx, q_indptr=indptr, max_rows=rows,
                                    kv_scale=cpu.kv_scale)
    for splits in (1, 2):
        got = attention.paged_attention(qg[-rows:], gpu.k[0], gpu.v[0], idx.cuda(), ctx.cuda(), q_indptr=indptr.cuda(),
                                        max_rows=rows, kv_scale=gpu.kv_scale, splits=splits)
        _close(got, ref, 2e-2)
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0
