"""3-bit weight formats: quantisation error, tile packing, codebook planes."""
import torch

from hibana_b200.ops.w3gemm import W3Linear
from hibana_b200.weights import w3


def test_int3g64_quantise_pack_and_linear_cpu():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(200, 256, generator=g) * 0.05
    q = w3.Int3G64.quantize(w)
    d = q.dequantize()
    assert float((d - w).abs().max()) <= float(q.scale.float().max()) * 0.75     # within ~half a step + bf16 rounding
    t = q.tiles()
    assert t.shape == (2, 4, w3.TILE_BYTES) and t.dtype == torch.uint8
    # decode one tile with the documented bit layout
    tile = t[1, 2]
    b = tile[:128 * 28].view(128, 7, 4).to(torch.int64)
    words = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    cols = []
    for wi in range(7):
        for i in range(5):
            cols += [(words[:, wi] >> (3 * i)) & 7, (words[:, wi] >> (3 * i + 16)) & 7]
    dec = torch.stack(cols, 1)[:, :64]
    want = torch.zeros(128, 64, dtype=torch.int64)
    want[:72] = q.codes[128:200, 128:192].long()
    assert torch.equal(dec, want)
    sz = tile[128 * 28:].view(128, 4).view(torch.bfloat16).view(128, 2)
    assert torch.equal(sz[:72, 0], q.scale[128:200, 2])
    lin = W3Linear(q)
    x = torch.randn(3, 256, generator=g).bfloat16()
    y = lin(x)
    assert torch.allclose(y.float(), x.float() @ d.to(torch.bfloat16).float().t(), atol=2e-2, rtol=2e-2)


def test_codebook_planes_roundtrip():
    g = torch.Generator().manual_seed(1)
    codes = torch.randint(0, 8, (64, 128), generator=g).to(torch.uint8)
    scales = (torch.rand(64, 4, generator=g) + 0.5).to(torch.float8_e4m3fn)
    row = torch.rand(64, generator=g) + 0.1
    levels = [-1.0, -0.62, -0.33, -0.1, 0.1, 0.33, 0.62, 1.0]
    cb = w3.CodebookW3.pack(codes, scales, row, levels)
    assert torch.equal(cb.codes(), codes)
    d = cb.dequantize()
    want = torch.tensor(levels)[codes.long()] * (scales.float() * row[:, None]).repeat_interleave(32, 1)
    assert torch.allclose(d, want)
    refit = cb.to_int3g64().dequantize()
    assert float((refit - d).abs().mean() / d.abs().mean()) < 0.25


def test_codebook_fit_beats_uniform_levels_and_gptq_beats_rounding():
    """Calibration tools: Lloyd codebook vs plain int3 on bell-shaped weights; GPTQ vs round-to-nearest on the
    layer output error with correlated inputs."""
    import torch
    from hibana_b200.weights import w3_calibrate as cal
    from hibana_b200.weights.w3 import Int3G64
    g = torch.Generator().manual_seed(0)
    w = torch.randn(96, 256, generator=g) * 0.05
    cb = cal.fit_codebook(w)
    assert cb.codes().max() <= 7 and len(cb.codebook) == 8
    err_cb = (cb.dequantize() - w).norm() / w.norm()
    err_rt = (Int3G64.quantize(w).dequantize() - w).norm() / w.norm()
    assert err_cb < 0.25 and err_cb < err_rt * 1.05, (float(err_cb), float(err_rt))
    # correlated activations: a few strong directions
    basis = torch.randn(256, 16, generator=g)
    x = torch.randn(512, 16, generator=g) @ basis.t() + 0.1 * torch.randn(512, 256, generator=g)
    h = cal.collect_hessian([x[:256], x[256:]], 256)
    q = cal.gptq_int3g64(w, h)
    e_gptq = cal.layer_error(w, q.dequantize(), x)
    e_rtn = cal.layer_error(w, Int3G64.quantize(w).dequantize(), x)
    assert e_gptq < e_rtn, (e_gptq, e_rtn)
    # the Hessian-weighted codebook is at least as good on the outputs as the unweighted one
    cbw = cal.fit_codebook(w, hessian_diag=torch.diag(h))
    assert cal.layer_error(w, cbw.dequantize(), x) < cal.layer_error(w, cb.dequantize(), x) * 1.1
