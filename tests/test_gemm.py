"""tcgen05 GEMM and NVFP4 quantiser against plain PyTorch fp32 references."""
import pytest
import torch

from hibana_b200 import _native as nv
from hibana_b200.ops import gemm, nvfp4


def test_e2m1_round_trip_cpu():
    codes = torch.arange(16, dtype=torch.int32)
    vals = nvfp4.e2m1_values(codes)
    assert torch.equal(nvfp4.e2m1_codes(vals) & 7, codes & 7)
    # ties go to the even mantissa
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert nvfp4.e2m1_values(nvfp4.e2m1_codes(x)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]


def test_swizzle_round_trip_cpu():
    sf = torch.randint(0, 255, (200, 20), dtype=torch.uint8)
    blocks = nvfp4.swizzle_sf(sf)
    assert blocks.shape == (2, 8, 512)
    assert torch.equal(nvfp4.unswizzle_sf(blocks, 200, 20), sf)
    r, g = 133, 7
    assert blocks[r // 128, g // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4] == sf[r, g]


def test_quant_dequant_error_cpu():
    x = torch.randn(64, 256)
    gs = float(x.abs().max()) / (6 * 448)
    q, sfb = nvfp4.quantize_ref(x, gs)
    y = nvfp4.dequantize_ref(q, sfb, gs)
    rel = (x - y).norm() / x.norm()
    assert rel < 0.12


def test_linear_nvfp4_cpu_reference():
    w = torch.randn(96, 128) * 0.02
    x = torch.randn(5, 128)
    wq = nvfp4.quantize_weight(w)
    gs = torch.tensor(float(x.abs().max()) / (6 * 448))
    xq = nvfp4.quantize(x.bfloat16(), gs)
    y = gemm.linear_nvfp4(xq, wq, gs * wq.gscale)
    ref = x @ w.t()
    assert (y.float() - ref).norm() / ref.norm() < 0.2


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (8, 5120, 5120), (64, 1024, 17408), (200, 384, 704),
                                   (300, 512, 1024), (1024, 2048, 4096)])
@pytest.mark.parametrize("epi", [gemm.EPI_STORE, gemm.EPI_RESIDUAL, gemm.EPI_SILU_MUL, gemm.EPI_STORE_F32])
def test_gemm_bf16(m, n, k, epi):
    dev = torch.device("cuda")
    x = (torch.randn(m, k, device=dev) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=dev) * 0.05).bfloat16()
    res = torch.randn(m, n, device=dev).bfloat16() if epi == gemm.EPI_RESIDUAL else None
    y = gemm.linear_bf16(x, w, epilogue=epi, residual=res)
    ref = gemm._ref_epilogue(x.float() @ w.float().t(), epi, res)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    err = (y.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    assert err <= 2e-2 * scale + 1e-3, (err, scale)


@pytest.mark.gpu
@pytest.mark.parametrize("m,k", [(1, 256), (7, 5120), (130, 704), (512, 17408)])
@pytest.mark.parametrize("mode", [nvfp4.MODE_PLAIN, nvfp4.MODE_SILU_SPLIT, nvfp4.MODE_SILU_PAIRS])
def test_quant_nvfp4_matches_reference(m, k, mode):
    dev = torch.device("cuda")
    cols = k if mode == nvfp4.MODE_PLAIN else 2 * k
    x = torch.randn(m, cols, device=dev).bfloat16()
    gs = torch.tensor(4.0 / (6 * 448), device=dev)
    got = nvfp4.quantize(x, gs, mode)
    y = x if mode == nvfp4.MODE_PLAIN else nvfp4._silu_mul(x, mode)
    packed, sfb = nvfp4.quantize_ref(y, gs)
    sf_got = nvfp4.unswizzle_sf(got.sf, m, k // 16)
    # silu uses __expf on the device: allow a handful of one-step differences in the fused modes
    mism_sf = (sf_got != sfb).float().mean().item()
    mism_q = (got.q != packed).float().mean().item()
    if mode == nvfp4.MODE_PLAIN:
        assert mism_sf == 0 and mism_q == 0
    else:
        assert mism_sf < 1e-3 and mism_q < 1e-2
    # padding scales are zero
    blocks = got.sf
    full = nvfp4.unswizzle_sf(blocks, blocks.shape[0] * 128, blocks.shape[1] * 4)
    assert full[m:].sum() == 0 and full[:, k // 16:].sum() == 0


@pytest.mark.gpu
def test_norm_quant_matches_reference():
    dev = torch.device("cuda")
    m, k = 37, 5120
    x = torch.randn(m, k, device=dev).bfloat16()
    res = torch.randn(m, k, device=dev).bfloat16()
    w = (torch.randn(k, device=dev) * 0.1 + 1).bfloat16()
    gs = torch.tensor(8.0 / (6 * 448), device=dev)
    res_ref = res.clone()
    ref_q, ref_y = nvfp4.rmsnorm_quantize(x.cpu(), w.cpu(), 1e-6, gs.cpu(), residual=(res_cpu := res_ref.cpu()),
                                          want_normed=True)
    got_q, got_y = nvfp4.rmsnorm_quantize(x, w, 1e-6, gs, residual=res, want_normed=True)
    assert torch.equal(res.cpu(), res_cpu)
    assert (got_y.cpu().float() - ref_y.float()).abs().max() < 0.05
    a, b = got_q.dequantize().cpu(), ref_q.dequantize()
    assert (a - b).norm() / b.norm() < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (4, 5120, 5120), (16, 1024, 17408), (64, 34816, 5120),
                                   (200, 384, 768), (300, 512, 1024), (1024, 5120, 2560), (2048, 768, 640)])
def test_gemm_nvfp4(m, n, k):
    dev = torch.device("cuda")
    x = torch.randn(m, k, device=dev).bfloat16()
    w = torch.randn(n, k, device=dev) * 0.02
    wq = nvfp4.quantize_weight(w)
    gs = torch.tensor(float(x.float().abs().max()) / (6 * 448), device=dev)
    xq = nvfp4.quantize(x, gs)
    alpha = (gs * wq.gscale).reshape(1)
    y = gemm.linear_nvfp4(xq, wq, alpha)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    ref = xq.dequantize() @ wq.dequantize().t()
    err = (y.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1.5e-2 * scale + 1e-4, (err, scale)


@pytest.mark.gpu
def test_gemm_nvfp4_epilogues_and_splitk_deterministic():
    dev = torch.device("cuda")
    m, n, k = 8, 1024, 8192
    x = torch.randn(m, k, device=dev).bfloat16()
    wq = nvfp4.quantize_weight(torch.randn(n, k, device=dev) * 0.02)
    gs = torch.tensor(float(x.float().abs().max()) / (6 * 448), device=dev)
    xq = nvfp4.quantize(x, gs)
    alpha = (gs * wq.gscale).reshape(1)
    acc = xq.dequantize() @ wq.dequantize().t()
    res = torch.randn(m, n, device=dev).bfloat16()
    for epi in (gemm.EPI_RESIDUAL, gemm.EPI_SILU_MUL):
        y1 = gemm.linear_nvfp4(xq, wq, alpha, epilogue=epi, residual=res, splits=4)
        y2 = gemm.linear_nvfp4(xq, wq, alpha, epilogue=epi, residual=res, splits=4)
        y3 = gemm.linear_nvfp4(xq, wq, alpha, epilogue=epi, residual=res, splits=1)
        ref = gemm._ref_epilogue(acc, epi, res)
        assert torch.equal(y1, y2)
        for y in (y1, y3):
            assert (y.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max() + 1e-3
    assert nv.read_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (4, 1280, 2560), (64, 768, 1152), (300, 640, 512), (2048, 1024, 2048)])
@pytest.mark.parametrize("dynamic", [False, True])
def test_fp8_gemm_matches_reference(m, n, k, dynamic):
    """e4m3 x e4m3 on tcgen05 (kind::f8f6f4) vs the fp32 product of the dequantised operands."""
    from hibana_b200.ops import fp8
    g = torch.Generator().manual_seed(m + n)
    x = (torch.randn(m, k, generator=g) * 1.5).bfloat16()
    w = fp8.Fp8Weight.quantize(torch.randn(n, k, generator=g) * 0.05)
    wc = fp8.Fp8Weight(w.q.cuda(), w.scale.cuda())
    if dynamic:
        q_ref, s_ref = fp8.quantize_rows(x)
        q, s = fp8.quantize_rows(x.cuda())
        assert torch.allclose(s.cpu(), s_ref, rtol=1e-3)
        ref = fp8.linear_fp8(q.cpu(), w, row_scales=s.cpu())
        got = fp8.linear_fp8(q, wc, row_scales=s)
    else:
        scale = torch.tensor([float(x.float().abs().max()) / 448.0])
        q = fp8.quantize_static(x.cuda(), scale.cuda())
        assert torch.equal(q.cpu().float(), fp8.quantize_static(x, scale).float())
        ref = fp8.linear_fp8(q.cpu(), w, x_scale=scale)
        got = fp8.linear_fp8(q, wc, x_scale=scale.cuda())
    err = (got.float().cpu() - ref.float()).abs().max() / ref.float().abs().max()
    assert float(err) < 1e-2, float(err)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (8, 1280, 2560), (64, 640, 4352), (130, 300, 512), (256, 1024, 1024)])
def test_w3_dequant_fused_gemm(m, n, k):
    """3-bit codes expanded in shared memory and multiplied on tcgen05 vs fp32 over the dequantised matrix."""
    from hibana_b200.ops.w3gemm import W3Linear
    g = torch.Generator().manual_seed(k + m)
    w = torch.randn(n, k, generator=g) * 0.05
    x = torch.randn(m, k, generator=g).bfloat16()
    lin = W3Linear.from_weight(w, "cuda")
    ref = x.float() @ lin.w3.dequantize().t()
    got = lin(x.cuda()).float().cpu()
    err = (got - ref).abs().max() / ref.abs().max()
    assert float(err) < 1e-2, float(err)
    res = torch.randn(m, n, generator=g).bfloat16()
    got = lin(x.cuda(), epilogue=1, residual=res.cuda()).float().cpu()
    assert float((got - (ref + res.float())).abs().max() / ref.abs().max()) < 2e-2
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (7, 1024, 5120), (64, 4352, 5120), (64, 34816, 1024), (100, 512, 768),
                                   (300, 192, 512), (300, 96, 512), (384, 4352, 1024), (1000, 2176, 768), (2048, 1024, 512)])
def test_silu_mul_requant_epilogue_matches_two_kernels(m, n, k):
    """gate/up GEMM with the SiLU-mul + NVFP4 requant epilogue == the SiLU-mul GEMM followed by the quantiser,
    byte for byte (packed values and every scale byte of real rows), for unsplit and cluster split-K launches and
    for prefill-sized calls (more than 256 rows: tokens on the 128-row side of the MMA); and the dequantised result is close to the fp32 reference of the same op."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(m * 7 + n)
    w = torch.randn(n, k, device=dev, generator=g) * 0.05
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    wq = nvfp4.quantize_weight(w)
    gs = torch.tensor(6.0 / (6 * 448), device=dev)
    xq = nvfp4.quantize(x, gs)
    alpha = (gs * wq.gscale).reshape(1)
    acc = xq.dequantize() @ wq.dequantize().t()
    ref = torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]
    out_scale = (ref.abs().max() / (6 * 448)).reshape(()).float()      # no clipping: the error is rounding only
    two = nvfp4.quantize(gemm.linear_nvfp4(xq, wq, alpha, epilogue=gemm.EPI_SILU_MUL), out_scale)
    one = gemm.linear_nvfp4_silu_quant(xq, wq, alpha, out_scale)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert torch.equal(one.q, two.q)
    groups = n // 2 // 16
    assert torch.equal(nvfp4.unswizzle_sf(one.sf, m, groups), nvfp4.unswizzle_sf(two.sf, m, groups))
    err = (one.dequantize() - ref).norm() / ref.norm().clamp_min(1e-6)
    assert err < 0.15, err
    # a second call reuses the persistent buffers and must give the same bytes (captured graphs replay it)
    again = gemm.linear_nvfp4_silu_quant(xq, wq, alpha, out_scale)
    assert torch.equal(again.q, two.q)
