"""3-bit weight formats: quantisation error, tile packing, codebook planes."""
import pytest
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


def test_reference_directory_round_trip_checksums_and_exact_serving(tmp_path):
    """The reference's on-disk 3-bit format (fragment-ordered bit planes, e4m3 group scales, row scales, manifest
    with SHA-256): written and read back bit for bit, a flipped byte is caught, tensor-parallel row ranges load, and
    the served projection equals the dequantised matrix without any re-fit."""
    import json
    import torch
    from hibana_b200.weights.w3 import CodebookW3
    from hibana_b200.weights import w3_reference as ref
    g = torch.Generator().manual_seed(0)
    lloyd = (-3.5, -2.25, -1.25, -0.40625, 0.40625, 1.25, 2.25, 3.5)
    n, k = 256, 384
    codes = torch.randint(0, 8, (n, k), generator=g)
    scales = (torch.rand(n, k // 32, generator=g) * 200 + 1).to(torch.float8_e4m3fn)
    row_scale = torch.rand(n, generator=g) * 1e-3 + 1e-4
    w = CodebookW3.pack(codes, scales, row_scale, lloyd)
    two = CodebookW3.pack(torch.randint(0, 4, (128, 128), generator=g), scales[:128, :4].contiguous(),
                          row_scale[:128], (-1.5, -0.4375, 0.4375, 1.5))
    d = ref.write_directory(tmp_path / "ckpt", {"layers.0.mlp.down": w, "draft.head": two}, revision="rev1")
    planes = ref.encode_planes(codes)
    assert planes.shape == (n // 32, k // 128, 3, 32, 4) and planes.dtype == torch.uint32
    # one element by hand: row 32*1 + 8*2 + 5, column 128*2 + 16*6 + 4*3 + 1 -> lane 4*5 + 3, tile 2, bit 4*1 + b + 18
    r, c = 32 + 16 + 5, 256 + 96 + 12 + 1
    for b in range(3):
        word = int(planes[1, 2, b, 23, 2].to(torch.int64)) & 0xFFFFFFFF
        assert (word >> ((4 + b + 18) % 32)) & 1 == (int(codes[r, c]) >> b) & 1
    ck = ref.ReferenceW3Checkpoint(d, revision="rev1")
    assert ck.names() == ["draft.head", "layers.0.mlp.down"]
    ck.verify()
    got = ck.load("layers.0.mlp.down")
    assert torch.equal(got.codes(), w.codes()) and torch.equal(got.scales, w.scales)
    assert torch.equal(got.row_scale, w.row_scale) and tuple(got.codebook) == lloyd
    assert torch.equal(ck.load("draft.head").dequantize(), two.dequantize())
    part = ck.load("layers.0.mlp.down", rows=slice(64, 192))
    assert torch.equal(part.dequantize(), w.dequantize()[64:192])
    lin = ref.CodebookLinear(got)
    x = torch.randn(5, k, generator=g).bfloat16()
    want = x.float() @ w.dequantize().t()
    assert (lin(x).float() - want).abs().max() <= 1e-2 * want.abs().max()
    with pytest.raises(ValueError):
        ref.ReferenceW3Checkpoint(d, revision="other")
    f = d / json.loads((d / "manifest.json").read_text())["weights"]["draft.head"]["file"]
    raw = bytearray(f.read_bytes())
    raw[-1] ^= 1
    f.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="checksum"):
        ck.load("draft.head")
    assert ref.current_checkpoint(tmp_path, "qwen38") is None
    (tmp_path / "qwen38-current").symlink_to(d)
    assert ref.current_checkpoint(tmp_path, "qwen38") == d.resolve()


def test_model_calibration_capture_fit_write_attach_cpu(tmp_path):
    """The whole calibration loop on the tiny dense model: covariances captured on the serving path, GPTQ fits that
    beat round-to-nearest on them, a digest-checked directory, and the engine decoding with the calibrated copies."""
    import json
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled
    from hibana_b200.weights import calibrate_model as cm
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    samples = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (96, 80, 120)]
    cov = cm.capture(model, samples, max_batch=2)
    names = [lin.name for lin in model.linears()]
    assert set(cov.matrices) == set(names)
    assert cov.rows["l0.qkv"] == sum(len(s) for s in samples)            # every prompt row, once
    assert cov.matrices["l0.down"].shape == (t.ffn, t.ffn)
    fitted, report = cm.fit(model, cov)
    assert set(fitted) == set(names)
    assert all(r["error_gptq"] < r["error_nearest"] for r in report), report
    d = cm.write_directory(tmp_path / "w3", fitted, target=t.name, report=report)
    back = cm.load_directory(d)
    assert all(torch.equal(back[n].codes, fitted[n].codes) and torch.equal(back[n].scale, fitted[n].scale)
               and torch.equal(back[n].zero, fitted[n].zero) for n in names)
    served = DenseModel(t, "cpu", seed=0)
    served.attach_w3()
    before = served.layers[0].qkv.w3.dense().clone()
    assert cm.attach(served, d, strict=True) == len(names)
    after = served.layers[0].qkv.w3.dense()
    assert not torch.equal(before, after) and torch.allclose(after.float(), fitted["l0.qkv"].dequantize(), atol=1e-6)
    out = Executor(served, max_batch=2, max_ctx=160, use_graphs=False).generate_batch(samples[:2], SamplingParams(max_tokens=6))
    assert all(len(r.output_ids) == 6 for r in out)
    # a damaged file is refused; names the model lacks are refused when asked to be strict
    manifest = json.loads((d / cm.MANIFEST).read_text())
    victim = d / manifest["weights"]["l1.o"]["file"]
    raw = bytearray(victim.read_bytes())
    raw[-1] ^= 0xFF
    victim.write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        cm.load_directory(d)
    cm.write_directory(tmp_path / "other", {"nowhere.proj": fitted["l0.o"]})
    with pytest.raises(ValueError):
        cm.attach(served, tmp_path / "other", strict=True)
    assert cm.attach(served, tmp_path / "other") == 0
    # the command-line driver end to end (two blocks of the tiny target, samples from a file)
    (tmp_path / "samples.json").write_text(json.dumps({"samples": samples[:2]}))
    cm.main(["--target", "dense-tiny", "--inputs", str(tmp_path / "samples.json"), "--output", str(tmp_path / "cli"),
             "--device", "cpu", "--layers", "1"])
    assert set(cm.load_directory(tmp_path / "cli")) == {"l0.qkv", "l0.o", "l0.gate_up", "l0.down"}


def test_routed_expert_calibration_capture_fit_attach_cpu(tmp_path):
    """Routed experts of a hybrid MoE model: per-expert covariances of the rows routed to each expert (both matrices),
    GPTQ per expert where enough rows were seen, stacks written next to the projections' and handed to the layers."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import scaled, tiny_hybrid_moe
    from hibana_b200.weights import calibrate_model as cm
    t = scaled(tiny_hybrid_moe(), expert_ffn=128, mtp_layers=0, mtp_depth=0, weight_format="bf16")
    model = HybridModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    samples = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (160, 140, 180, 150)]
    cov = cm.capture(model, samples, max_batch=2)
    ec = cov.experts
    layers = cm.expert_layers(model)
    assert layers and set(ec.h1) == set(layers)
    name = next(iter(layers))
    ew = layers[name].experts
    rows = sum(len(s) for s in samples)
    assert int(ec.rows[name].sum()) == rows * t.top_k                      # every (token, choice) pair, once
    assert ec.h1[name].shape == (ew.experts, ew.hidden, ew.hidden) and ec.h2[name].shape == (ew.experts, ew.inter, ew.inter)
    e = int(ec.rows[name].argmax())
    assert torch.allclose(ec.h1[name][e], ec.h1[name][e].t(), atol=1e-3) and float(ec.h1[name][e].diagonal().min()) >= 0
    efit, ereport = cm.fit_experts(model, ec, min_rows=64)
    assert set(efit) == {f"{n}.fc{w}" for n in layers for w in (1, 2)}
    r0 = next(r for r in ereport if r["name"] == name)
    assert r0["calibrated"] >= 1
    assert r0["fc1_error_gptq"] < r0["fc1_error_nearest"] and r0["fc2_error_gptq"] < r0["fc2_error_nearest"], r0
    assert efit[f"{name}.fc1"].shape == (ew.experts * ew.n1, ew.hidden)
    fitted, report = cm.fit(model, cov)
    fitted.update(efit)
    d = cm.write_directory(tmp_path / "w3", fitted, target=t.name, report=report + ereport)
    served = HybridModel(t, "cpu", seed=0)
    served.attach_w3()
    before = layers and cm.expert_layers(served)[name].experts_w3.dense(1).clone()
    n = cm.attach(served, d, strict=True)
    assert n == len(fitted) - len(layers)                                   # fc1 + fc2 of a layer attach as one
    after = cm.expert_layers(served)[name].experts_w3.dense(1)
    assert not torch.equal(before, after)
    assert torch.allclose(after.reshape(-1, ew.hidden).float(), efit[f"{name}.fc1"].dequantize().float(), atol=1e-6)
    out = Executor(served, max_batch=2, max_ctx=200, use_graphs=False).generate_batch(samples[:2], SamplingParams(max_tokens=4))
    assert all(len(r.output_ids) == 4 for r in out)
