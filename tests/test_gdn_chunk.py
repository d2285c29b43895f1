"""Chunked (WY) gated delta rule against the sequential fp32 reference."""
import pytest
import torch

from hibana_b200.ops import gdn_chunk, recurrent


def _case(rows, k_heads, v_heads, kdim, vdim, seed=0, slots=6):
    g = torch.Generator().manual_seed(seed)
    t = sum(rows)
    q = torch.randn(t, k_heads * kdim, generator=g).bfloat16()
    k = torch.randn(t, k_heads * kdim, generator=g).bfloat16()
    v = torch.randn(t, v_heads * vdim, generator=g).bfloat16()
    gl = -torch.rand(t, v_heads, generator=g) * 0.3          # log decay
    beta = torch.rand(t, v_heads, generator=g)
    state = torch.randn(slots, v_heads, vdim, kdim, generator=g) * 0.1
    indptr = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    slot_in = torch.arange(len(rows), dtype=torch.int32)
    slot_out = slot_in + len(rows)
    return q, k, v, gl, beta, state, indptr, slot_in, slot_out


@pytest.mark.parametrize("rows", [[130], [64, 1, 200], [63, 65]])
@pytest.mark.parametrize("heads", [(2, 4, 32, 32), (1, 2, 64, 64)])
def test_chunked_matches_sequential_cpu(rows, heads):
    kh, vh, kd, vd = heads
    q, k, v, gl, beta, state, indptr, sin, sout = _case(rows, kh, vh, kd, vd)
    has_init = torch.tensor([1, 0, 1][:len(rows)], dtype=torch.int32)
    st_ref = state.clone()
    ref = recurrent.gdn_scan(q, k, v, gl, beta, st_ref, sin, sout, k_heads=kh, v_heads=vh, kdim=kd, vdim=vd,
                             q_indptr=indptr, has_init=has_init)
    st = state.clone()
    ranges = recurrent._ranges(indptr, len(rows))
    got = gdn_chunk.gdn_chunked(q, k, v, gl, beta, st, sin, sout, k_heads=kh, v_heads=vh, kdim=kd, vdim=vd,
                                scale=kd ** -0.5, l2norm=True, ranges=ranges, has_init=has_init.tolist())
    assert torch.allclose(got.float(), ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(st, st_ref, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [[300], [128, 70, 513]])
def test_chunked_gpu_matches_sequential(rows):
    """Phase 1 in batched GEMMs + the mma.sync state pass against the fp32 sequential reference (head dim 128)."""
    kh, vh, kd, vd = 2, 4, 128, 128
    q, k, v, gl, beta, state, indptr, sin, sout = _case(rows, kh, vh, kd, vd, seed=3)
    has_init = torch.tensor([1, 0, 1][:len(rows)], dtype=torch.int32)
    st_ref = state.clone()
    ref = recurrent.gdn_scan(q, k, v, gl, beta, st_ref, sin, sout, k_heads=kh, v_heads=vh, kdim=kd, vdim=vd,
                             q_indptr=indptr, has_init=has_init)
    st = state.cuda()
    got = recurrent.gdn_scan(q.cuda(), k.cuda(), v.cuda(), gl.cuda(), beta.cuda(), st, sin.cuda(), sout.cuda(),
                             k_heads=kh, v_heads=vh, kdim=kd, vdim=vd, q_indptr=indptr.cuda(),
                             has_init=has_init.cuda(), host_rows=rows)
    err = (got.float().cpu() - ref.float()).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.float().abs().max().item()), err
    assert torch.allclose(st.cpu(), st_ref, atol=2e-2, rtol=2e-2)
    # the token-serial kernel and the chunked form agree on the GPU as well
    st2 = state.cuda()
    seq = recurrent.gdn_scan(q.cuda(), k.cuda(), v.cuda(), gl.cuda(), beta.cuda(), st2, sin.cuda(), sout.cuda(),
                             k_heads=kh, v_heads=vh, kdim=kd, vdim=vd, q_indptr=indptr.cuda(),
                             has_init=has_init.cuda())
    assert (seq.float() - got.float()).abs().max().item() < 3e-2 * max(1.0, ref.float().abs().max().item())


def _mamba_case(rows, heads, groups, p, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = sum(rows)
    x = torch.randn(t, heads * p, generator=g).bfloat16()
    bm = (torch.randn(t, groups * n, generator=g) * 0.3).bfloat16()
    cm = (torch.randn(t, groups * n, generator=g) * 0.3).bfloat16()
    dt = torch.randn(t, heads, generator=g).bfloat16()
    a_log = torch.rand(heads, generator=g)
    dt_bias = torch.randn(heads, generator=g) * 0.1
    dskip = torch.randn(heads, generator=g)
    state = torch.randn(2 * len(rows), heads, p, n, generator=g) * 0.1
    indptr = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32)
    sin = torch.arange(len(rows), dtype=torch.int32)
    return x, bm, cm, dt, a_log, dt_bias, dskip, state, indptr, sin, sin + len(rows)


@pytest.mark.parametrize("rows", [[150], [64, 3, 129]])
def test_ssd_chunked_matches_sequential_cpu(rows):
    from hibana_b200.ops import ssd_chunk
    heads, groups, p, n = 4, 2, 32, 16
    x, bm, cm, dt, a_log, dtb, dsk, state, indptr, sin, sout = _mamba_case(rows, heads, groups, p, n)
    has_init = torch.tensor([1, 0, 1][:len(rows)], dtype=torch.int32)
    st_ref = state.clone()
    ref = recurrent.mamba2_scan(x, bm, cm, dt, a_log, dtb, dsk, st_ref, sin, sout, heads=heads, groups=groups,
                                head_dim=p, d_state=n, q_indptr=indptr, has_init=has_init)
    st = state.clone()
    got = ssd_chunk.mamba2_chunked(x, bm, cm, dt, a_log, dtb, dsk, st, sin, sout, heads=heads, groups=groups,
                                   head_dim=p, d_state=n, ranges=recurrent._ranges(indptr, len(rows)),
                                   has_init=has_init.tolist())
    assert torch.allclose(got.float(), ref.float(), atol=3e-2, rtol=3e-2)
    assert torch.allclose(st, st_ref, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [[300], [128, 70, 513]])
def test_ssd_chunked_gpu_matches_sequential(rows):
    heads, groups, p, n = 8, 2, 64, 128
    x, bm, cm, dt, a_log, dtb, dsk, state, indptr, sin, sout = _mamba_case(rows, heads, groups, p, n, seed=4)
    has_init = torch.tensor([1, 0, 1][:len(rows)], dtype=torch.int32)
    st_ref = state.clone()
    ref = recurrent.mamba2_scan(x, bm, cm, dt, a_log, dtb, dsk, st_ref, sin, sout, heads=heads, groups=groups,
                                head_dim=p, d_state=n, q_indptr=indptr, has_init=has_init)
    st = state.cuda()
    got = recurrent.mamba2_scan(x.cuda(), bm.cuda(), cm.cuda(), dt.cuda(), a_log.cuda(), dtb.cuda(), dsk.cuda(), st,
                                sin.cuda(), sout.cuda(), heads=heads, groups=groups, head_dim=p, d_state=n,
                                q_indptr=indptr.cuda(), has_init=has_init.cuda(), host_rows=rows)
    scale = max(1.0, ref.float().abs().max().item())
    assert (got.float().cpu() - ref.float()).abs().max().item() < 3e-2 * scale
    assert torch.allclose(st.cpu(), st_ref, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [64, 200])
def test_phase1_kernel_matches_batched_reference(n):
    """gdn_phase1_kernel (bf16 tensor-core products, fp32 triangular inverse) against the fp32 PyTorch phase 1."""
    kh, vh = 2, 4
    q, k, v, gl, beta, *_ = _case([n], kh, vh, 128, 128, seed=9)
    qkv = torch.cat([q, k, v], 1).cuda()                      # column slices of one buffer, as in the model
    qd, kd_, vd = qkv[:, :kh * 128], qkv[:, kh * 128:2 * kh * 128], qkv[:, 2 * kh * 128:]
    ref = gdn_chunk.prepare(qd, kd_, vd, gl.cuda(), beta.cuda(), k_heads=kh, v_heads=vh, kdim=128, vdim=128,
                            scale=128 ** -0.5, l2norm=True)
    got = gdn_chunk.prepare_native(qd, kd_, vd, gl.cuda(), beta.cuda(), k_heads=kh, v_heads=vh, scale=128 ** -0.5,
                                   l2norm=True)
    assert got["nc"] == ref["nc"]
    for name, tol in (("g_end", 1e-4), ("qg", 1e-2), ("kd", 1e-2), ("m", 2e-2), ("u", 3e-2), ("w", 3e-2)):
        a, b = got[name].float(), ref[name].float()
        err = (a - b).abs().max().item()
        assert err <= tol * max(1.0, b.abs().max().item()), (name, err, b.abs().max().item())
