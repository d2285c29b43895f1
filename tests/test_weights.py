"""Checkpoint round trips: ModelOpt NVFP4 tensors, sharded load, generation equality."""
import pytest
import torch

from hibana_b200.engine.executor import Executor
from hibana_b200.engine.request import SamplingParams
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled
from hibana_b200.weights import checkpoint, modelopt


def test_dense_checkpoint_roundtrip_and_tp_shards(tmp_path):
    t = scaled(dense_tiny(), weight_format="nvfp4")
    model = DenseModel(t, "cpu", seed=0)
    for lin in model.linears():
        lin.set_input_amax(4.0)
    checkpoint.save_dense(model, str(tmp_path), layers_per_file=1)
    loaded = checkpoint.load_dense(t, str(tmp_path))
    for a, b in zip(model.linears(), loaded.linears()):
        assert torch.equal(a.wq.q, b.wq.q) and torch.equal(a.wq.sf, b.wq.sf) and torch.equal(a.alpha, b.alpha)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, t.vocab, (20,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(max_tokens=5)
    a = [r.output_ids for r in Executor(model, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)]
    b = [r.output_ids for r in Executor(loaded, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)]
    assert a == b
    # a tensor-parallel shard read from the file equals the shard cut from the in-memory model
    ref = DenseModel.sharded(t, 2, 1, "cpu", seed=0)
    shard = checkpoint.load_dense(t, str(tmp_path), tp=2, rank=1)
    for x, y in zip(ref.linears(), shard.linears()):
        assert torch.equal(x.wq.q, y.wq.q) and torch.equal(x.wq.sf, y.wq.sf)


def test_hf_layout_checkpoint_with_separate_projections(tmp_path):
    """A checkpoint in the published layout (separate q/k/v and gate/up projections, row-major scales): loading
    fuses and interleaves them into the kernel-order matrices bit for bit, for the whole model and for a
    tensor-parallel shard, and mismatched per-tensor scales are refused."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    t = scaled(dense_tiny(), weight_format="nvfp4")
    model = DenseModel(t, "cpu", seed=0)
    for i, lin in enumerate(model.linears()):
        lin.set_input_amax(3.0 + i)
    checkpoint.save_dense(model, str(tmp_path), layers_per_file=1, hf_layout=True)
    snap = checkpoint.Snapshot(str(tmp_path))
    assert "model.layers.0.self_attn.q_proj.weight" in snap and "model.layers.0.self_attn.qkv_proj.weight" not in snap
    loaded = checkpoint.load_dense(t, str(tmp_path))
    for a, b in zip(model.linears(), loaded.linears()):
        assert torch.equal(a.wq.q, b.wq.q) and torch.equal(a.wq.sf, b.wq.sf) and torch.equal(a.alpha, b.alpha)
    ref = DenseModel.sharded(t, 2, 1, "cpu", seed=0)
    shard = checkpoint.load_dense(t, str(tmp_path), tp=2, rank=1)
    for x, y in zip(ref.linears(), shard.linears()):
        assert torch.equal(x.wq.q, y.wq.q) and torch.equal(x.wq.sf, y.wq.sf)
    # k_proj quantised with another per-tensor scale: fusing would need a requantisation, so the load refuses
    f = tmp_path / snap.map["model.layers.0.self_attn.k_proj.weight_scale_2"]
    with safe_open(str(f), framework="pt") as h:
        tensors = {k: h.get_tensor(k) for k in h.keys()}
    tensors["model.layers.0.self_attn.k_proj.weight_scale_2"] = tensors["model.layers.0.self_attn.k_proj.weight_scale_2"] * 2
    save_file(tensors, str(f))
    with pytest.raises(ValueError):
        checkpoint.load_dense(t, str(tmp_path))


def test_unpack_fp4():
    q = torch.tensor([[0x21, 0xF7]], dtype=torch.uint8)
    assert modelopt.unpack_fp4(q).tolist() == [[0.5, 1.0, 6.0, -6.0]]


def test_gguf_reader_and_block_codecs(tmp_path):
    """GGUF container round trip (metadata, alignment, tensor directory) and the Q8_0 / F16 / BF16 codecs; the IQ2
    decoders run against a synthetic lattice table and a hand-packed block."""
    import numpy as np
    from hibana_b200.weights import ggml
    rng = np.random.default_rng(0)
    w = rng.standard_normal((6, 64)).astype(np.float32)
    h = rng.standard_normal((3, 5)).astype(np.float16)
    bf = (rng.standard_normal(8).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    path = str(tmp_path / "t.gguf")
    ggml.write_gguf(path, {"a.weight": (ggml.quantize_q8_0(w), ggml.T_Q8_0, (6, 64)),
                           "b": (h.view(np.uint8).reshape(-1), ggml.T_F16, (3, 5)),
                           "c": (bf.view(np.uint8), ggml.T_BF16, (8,))},
                    meta={"general.architecture": "test", "block_count": 7})
    f = ggml.GgufFile(path)
    assert f.meta["general.architecture"] == "test" and f.meta["block_count"] == 7 and f.version == 3
    assert f.tensors["a.weight"].shape == (6, 64) and f.tensors["a.weight"].nbytes == 6 * 2 * 34
    got = f.load("a.weight")
    assert np.abs(got - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-3          # half a quantisation step
    assert np.array_equal(f.load("b"), h.astype(np.float32))
    assert np.array_equal(f.load("c"), (bf.astype(np.uint32) << 16).view(np.float32))
    f.close()
    # IQ2_XXS: one super-block, all indices -> entry 3 of a synthetic grid, sub-scale 5, signs pattern 0b0000101
    grid = rng.integers(1, 44, size=(256, 8)).astype(np.uint8)
    blk = np.zeros(66, dtype=np.uint8)
    blk[:2] = np.float16(0.5).reshape(1).view(np.uint8)
    words = np.zeros((8, 2), dtype=np.uint32)
    words[:, 0] = 3 | (3 << 8) | (3 << 16) | (3 << 24)
    sidx = 0b0000101
    words[:, 1] = sidx | (sidx << 7) | (sidx << 14) | (sidx << 21) | (5 << 28)
    blk[2:] = words.view(np.uint8).reshape(-1)
    out = ggml.dequantize(blk, ggml.T_IQ2_XXS, (256,), grids={"iq2_xxs": grid})
    signs = np.array([-1, 1, -1, 1, 1, 1, 1, 1], dtype=np.float32)              # bits 0 and 2 set; parity even -> bit 7 clear
    expect = np.tile(grid[3].astype(np.float32) * signs * 0.5 * (0.5 + 5) * 0.25, 32)
    assert np.allclose(out, expect)
    with pytest.raises(ValueError):
        ggml.dequantize(blk, ggml.T_IQ2_XXS, (256,))


@pytest.mark.parametrize("family", ["tiny", "flashnext"])
def test_hybrid_snapshot_roundtrip_and_serving_from_weights(tmp_path, family):
    """Snapshots of hybrid models: every tensor (quantised linears, expert stacks, convolution / recurrence
    parameters, MTP head) comes back bit for bit, `weights=<dir>` builds the same model through the engine, and a
    tensor-parallel rank round-trips its own shard."""
    from hibana_b200 import config as cfgmod
    from hibana_b200.engine.llm import LLM
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import get_target
    from hibana_b200.weights import snapshot
    t = get_target(family)
    if family != "tiny":
        t = scaled(t, layers=4, hidden=256, vocab=2048, q_heads=4, kv_heads=2, head_dim=64, gdn_k_heads=2,
                   gdn_v_heads=4, gdn_head_dim=64, experts=8, top_k=2, expert_ffn=128, shared_ffn=128, hyper_streams=0,
                   max_context=512, prefill_chunk=128, kv_dtype="bf16")
    t = scaled(t, weight_format="nvfp4")
    a = HybridModel(t, "cpu", seed=11)
    snapshot.save_state(a, str(tmp_path / "ckpt"))
    b = HybridModel(t, "cpu", seed=99)                           # different weights before loading
    n = snapshot.load_state(b, str(tmp_path / "ckpt"))
    ta, tb = snapshot.named_tensors(a), snapshot.named_tensors(b)
    assert n > 20 and set(ta) == set(tb)
    assert all(torch.equal(ta[k][2], tb[k][2]) for k in ta)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, t.vocab, (20,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(max_tokens=4)
    cfg = cfgmod.EngineConfig(max_batch=2, max_context=128, cuda_graphs=False, seed=5)
    want = [r.output_ids for r in LLM(cfg, target=t, device="cpu", model=a).generate(prompts, sp)]
    got = [r.output_ids for r in LLM(cfg.replace(weights=str(tmp_path / "ckpt")), target=t, device="cpu").generate(prompts, sp)]
    assert got == want
    shard = HybridModel.sharded(t, 2, 1, "cpu", seed=11)
    snapshot.save_state(shard, str(tmp_path / "tp"))
    other = HybridModel.sharded(t, 2, 1, "cpu", seed=3)
    snapshot.load_state(other, str(tmp_path / "tp"))
    ts, to = snapshot.named_tensors(shard), snapshot.named_tensors(other)
    assert all(torch.equal(ts[k][2], to[k][2]) for k in ts) and (tmp_path / "tp" / "rank1of2").is_dir()
    with pytest.raises(ValueError):
        snapshot.load_state(HybridModel(t, "cpu", seed=0), str(tmp_path / "tp" / "rank1of2"))


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4"])
def test_nemotron_checkpoint_layout_round_trip_cpu(tmp_path, fmt):
    """A Nemotron-class model written under the published checkpoint's tensor names (one mixer per block, q / k / v
    and the routed experts as separate tensors) loads back bit for bit: same tensors, same tokens."""
    import dataclasses
    import json
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import nemotron, scaled
    from hibana_b200.weights import nemotron_layout as nl
    base = nemotron()
    t = scaled(base, hidden=256, vocab=512, q_heads=4, kv_heads=2, head_dim=64, mamba_heads=8, mamba_head_dim=32,
               mamba_state=64, mamba_groups=2, experts=8, top_k=3, expert_ffn=128, shared_ffn=128, latent=128,
               weight_format=fmt, kv_dtype="bf16", mtp_layers=0, max_context=512)
    t = dataclasses.replace(t, layers=base.layers[:9])            # M E M E M E M * E: every kind of block
    model = HybridModel(t, "cpu", seed=3)
    d = nl.save(model, tmp_path / "ckpt", blocks_per_file=4)
    index = json.loads((d / "model.safetensors.index.json").read_text())["weight_map"]
    assert "language_model.backbone.layers.7.mixer.q_proj.weight" in index
    assert "language_model.backbone.layers.1.mixer.experts.7.down_proj.weight" in index
    assert "language_model.backbone.layers.0.mixer.conv1d.weight" in index and len(set(index.values())) == 4
    if fmt == "nvfp4":
        assert "language_model.backbone.layers.1.mixer.experts.0.up_proj.weight_scale_2" in index
    other = nl.load(t, d, "cpu", seed=99)                          # another seed: nothing may survive from init
    a, b = nl.tensors_of(model), nl.tensors_of(other)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k].view(torch.uint8) if a[k].dtype == torch.float8_e4m3fn else a[k],
                           b[k].view(torch.uint8) if b[k].dtype == torch.float8_e4m3fn else b[k]), k
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (24, 17)]
    sp = SamplingParams(max_tokens=6)
    want = [r.output_ids for r in Executor(model, max_batch=2, max_ctx=96, use_graphs=False).generate_batch(prompts, sp)]
    got = [r.output_ids for r in Executor(other, max_batch=2, max_ctx=96, use_graphs=False).generate_batch(prompts, sp)]
    assert got == want


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4"])
def test_qwen_checkpoint_layout_round_trip_cpu(tmp_path, fmt):
    """A Qwen3.8-class model written under the published checkpoint's tensor names (linear_attn / self_attn / mlp per
    layer, separate in_proj_qkv | in_proj_z, q | k | v and gate | up tensors, the prediction head under `mtp.`) loads
    back bit for bit through `load_hybrid`: same tensors, same tokens."""
    import json
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import qwen38_hybrid, scaled
    from hibana_b200.weights import qwen_layout as ql
    from hibana_b200.weights.checkpoint import load_hybrid
    t = scaled(qwen38_hybrid(), layers=4, hidden=256, vocab=512, q_heads=4, kv_heads=2, head_dim=64, ffn=512,
               gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=64, weight_format=fmt, kv_dtype="bf16", max_context=512)
    model = HybridModel(t, "cpu", seed=3)
    assert model.mtp is not None
    d = ql.save(model, tmp_path / "ckpt", layers_per_file=2)
    index = json.loads((d / "model.safetensors.index.json").read_text())["weight_map"]
    for name in ("model.language_model.layers.0.linear_attn.in_proj_qkv.weight",
                 "model.language_model.layers.0.linear_attn.in_proj_z.weight",
                 "model.language_model.layers.2.linear_attn.A_log",
                 "model.language_model.layers.3.self_attn.q_proj.weight",
                 "model.language_model.layers.3.self_attn.k_norm.weight",
                 "model.language_model.layers.1.mlp.gate_proj.weight", "mtp.fc.weight",
                 "mtp.layers.0.self_attn.o_proj.weight", "mtp.pre_fc_norm_hidden.weight"):
        assert name in index, name
    if fmt == "nvfp4":
        assert "model.language_model.layers.1.mlp.up_proj.weight_scale_2" in index
    other = load_hybrid(t, str(d), "cpu", seed=99)                 # another seed: nothing may survive from init
    a, b = ql.tensors_of(model), ql.tensors_of(other)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k].view(torch.uint8) if a[k].dtype == torch.float8_e4m3fn else a[k],
                           b[k].view(torch.uint8) if b[k].dtype == torch.float8_e4m3fn else b[k]), k
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (24, 17)]
    sp = SamplingParams(max_tokens=6)
    want = [r.output_ids for r in Executor(model, max_batch=2, max_ctx=96, use_graphs=False).generate_batch(prompts, sp)]
    got = [r.output_ids for r in Executor(other, max_batch=2, max_ctx=96, use_graphs=False).generate_batch(prompts, sp)]
    assert got == want


def test_qwen_checkpoint_layout_block_scaled_fp8_mixers_cpu(tmp_path):
    """Mixer projections stored as FP8 with one scale per 128 x 128 block (`weight_scale_inv`) load as the bf16
    expansion of exactly those values; the rest of the checkpoint is untouched."""
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import qwen38_hybrid, scaled
    from hibana_b200.weights import qwen_layout as ql
    w = torch.randn(200, 300, generator=torch.Generator().manual_seed(1)).bfloat16()
    q, s = ql.fp8_block_quant(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    back = ql.fp8_block_dequant(q, s)
    assert (back.float() - w.float()).abs().max() <= 0.07 * w.float().abs().max()
    q2, s2 = ql.fp8_block_quant(back)                              # a fixed point: stored values survive a round trip
    assert torch.equal(ql.fp8_block_dequant(q2, s2), back)
    t = scaled(qwen38_hybrid(), layers=4, hidden=256, vocab=512, q_heads=4, kv_heads=2, head_dim=64, ffn=512,
               gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=64, weight_format="bf16", kv_dtype="bf16", mtp_layers=0,
               max_context=512)
    model = HybridModel(t, "cpu", seed=5)
    d = ql.save(model, tmp_path / "ckpt", fp8_mixers=True)
    other = ql.load(t, d, "cpu", seed=9)
    lin, src = other.blocks[0].mixer.in_qkvz, model.blocks[0].mixer.in_qkvz
    qk, vd = 2 * 64, 4 * 64
    parts = [src.weight[:2 * qk + vd], src.weight[2 * qk + vd:]]
    want = torch.cat([ql.fp8_block_dequant(*ql.fp8_block_quant(p)) for p in parts], 0)
    assert lin.fmt == "bf16" and torch.equal(lin.weight, want)
    assert torch.equal(other.blocks[3].mixer.o.weight, ql.fp8_block_dequant(*ql.fp8_block_quant(model.blocks[3].mixer.o.weight)))
    assert torch.equal(other.blocks[1].ffn.down.weight, model.blocks[1].ffn.down.weight)
    assert torch.equal(other.blocks[2].mixer.conv_w, model.blocks[2].mixer.conv_w)
