"""GGML block formats served in place: the decode-fused kernels against the numpy decoders."""
import numpy as np
import pytest
import torch

from hibana_b200.ops import ggml as ops
from hibana_b200.weights import ggml as fmt


def _grid(entries, seed=1):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.choice(np.array([8, 25, 43], dtype=np.uint8), size=(entries, 8)))


def _case(name, n, k, dev):
    grid = None if name == "q8_0" else _grid(256 if name == "iq2_xxs" else 512)
    raw = ops.random_blocks(name, n, k, seed=3)
    return ops.PackedLinear(raw.to(dev), name, n, k, grid)


@pytest.mark.parametrize("name", ["q8_0", "iq2_xxs", "iq2_xs"])
def test_packed_linear_reference_path_cpu(name):
    lin = _case(name, 24, 512, "cpu")
    w = lin.dequantize().float()
    grids = {name: lin.grid.numpy()} if lin.grid is not None else None
    want = torch.from_numpy(fmt.dequantize(lin.raw.numpy().reshape(-1), lin.gtype, (24, 512), grids))
    assert torch.equal(w, want.to(torch.bfloat16).float())
    x = torch.randn(3, 512).bfloat16()
    y = lin(x)
    assert (y.float() - x.float() @ w.t()).abs().max() <= 2e-2 * (x.float() @ w.t()).abs().max() + 1e-3
    with pytest.raises(ValueError):
        ops.PackedLinear(lin.raw, name, 24, 500)                        # rows hold whole blocks
    if name != "q8_0":
        with pytest.raises(ValueError):
            ops.PackedLinear(lin.raw, name, 24, 512, None)              # no lattice table, no decoding


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["q8_0", "iq2_xxs", "iq2_xs"])
@pytest.mark.parametrize("m", [1, 3, 8, 40])
def test_packed_linear_kernels_match_decoders(name, m):
    n, k = 300, 1024
    cpu = _case(name, n, k, "cpu")
    gpu = _case(name, n, k, "cuda")
    w = cpu.dequantize().float()
    assert torch.equal(gpu.dequantize().float().cpu(), w)                # expansion kernel: bit-equal to numpy
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).bfloat16()
    want = x.float() @ w.t()
    got = gpu(x.cuda()).float().cpu()
    assert (got - want).abs().max() <= 1.5e-2 * want.abs().max() + 1e-3
    r2 = gpu(x.cuda(), relu2=True).float().cpu()
    assert (r2 - torch.relu(want) ** 2).abs().max() <= 3e-2 * (want ** 2).abs().max() + 1e-3


@pytest.mark.gpu
def test_packed_experts_grouped_decode_matches_reference():
    e, h, inter = 6, 512, 256
    grid = _grid(256)
    fc1 = ops.random_blocks("iq2_xxs", e * inter, h, seed=5, scale=0.01)
    fc2 = ops.random_blocks("q8_0", e * h, inter, seed=6, scale=0.002)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(5, h, generator=g).bfloat16()
    ids = torch.stack([torch.randperm(e, generator=g)[:2] for _ in range(5)]).int()
    wts = torch.rand(5, 2, generator=g)
    outs = []
    for dev in ("cpu", "cuda"):
        ex = ops.PackedExperts(ops.PackedLinear(fc1.to(dev), "iq2_xxs", e * inter, h, grid),
                               ops.PackedLinear(fc2.to(dev), "q8_0", e * h, inter), e)
        outs.append(ex.forward(x.to(dev), ids.to(dev), wts.to(dev)).float().cpu())
    assert (outs[0] - outs[1]).abs().max() <= 3e-2 * outs[0].abs().max() + 1e-3


@pytest.mark.gpu
def test_packed_experts_prefill_sized_matches_reference():
    """More (token, expert) pairs than the decode kernel takes: the expert stacks are expanded to bf16 once and the
    grouped tensor-core GEMMs run them; same result as the per-expert reference."""
    e, h, inter = 8, 512, 256
    grid = _grid(256)
    fc1 = ops.random_blocks("iq2_xxs", e * inter, h, seed=15, scale=0.01)
    fc2 = ops.random_blocks("q8_0", e * h, inter, seed=16, scale=0.002)
    g = torch.Generator().manual_seed(17)
    t, k = 1100, 4
    x = torch.randn(t, h, generator=g).bfloat16()
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).int()
    wts = torch.rand(t, k, generator=g)
    outs = []
    for dev in ("cpu", "cuda"):
        ex = ops.PackedExperts(ops.PackedLinear(fc1.to(dev), "iq2_xxs", e * inter, h, grid),
                               ops.PackedLinear(fc2.to(dev), "q8_0", e * h, inter), e)
        outs.append(ex.forward(x.to(dev), ids.to(dev), wts.to(dev)).float().cpu())
    assert (outs[0] - outs[1]).abs().max() <= 3e-2 * outs[0].abs().max() + 1e-3


def _small_bolt():
    from hibana_b200.target import bolt, scaled
    t = scaled(bolt(), layers=9, hidden=256, vocab=2048, q_heads=4, kv_heads=2, head_dim=64, mamba_heads=8,
               mamba_head_dim=32, mamba_state=64, mamba_groups=2, mamba_chunk=64, top_k=3, shared_ffn=256, latent=256,
               max_context=512, prefill_chunk=128, kv_dtype="bf16",
               moe_specs=((1, 6, 256), (3, 10, 512), (5, 6, 256), (8, 8, 256)))
    return t


def test_bolt_preset_and_heterogeneous_blocks_cpu():
    """The Bolt preset: 88 blocks (8 attention, 40 MoE with their own expert count / width, the rest Mamba-2); a
    scaled copy builds with per-block expert geometry in GGML blocks and decodes through the engine."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.bolt import BoltMoeLayer, GgmlLinear
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import ATTN, LATENT_MOE, bolt
    full = bolt()
    kinds = [f for _, f in full.layers]
    assert len(full.layers) == 88 and kinds.count(LATENT_MOE) == 40 and sum(m == ATTN for m, _ in full.layers) == 8
    assert full.block(48).experts == 496 and full.block(3).expert_ffn == 1536 and full.block(0).experts == 240
    t = _small_bolt()
    model = HybridModel(t, "cpu", seed=0)
    ffns = [b.ffn for b in model.blocks if b.ffn is not None]
    assert all(isinstance(f, BoltMoeLayer) for f in ffns)
    assert [f.experts.experts for f in ffns] == [6, 10, 6, 8] and ffns[1].experts.inter == 512
    assert isinstance(model.blocks[0].mixer.in_proj, GgmlLinear) and model.blocks[0].mixer.in_proj.fmt == "q8_0"
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (20, 9)]
    out = Executor(model, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, SamplingParams(max_tokens=5))
    assert all(len(r.output_ids) == 5 for r in out)
    again = Executor(model, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, SamplingParams(max_tokens=5))
    assert [r.output_ids for r in again] == [r.output_ids for r in out]


@pytest.mark.gpu
def test_bolt_decodes_on_gpu_with_graphs():
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    t = _small_bolt()
    model = HybridModel(t, "cuda:0", seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (20, 9)]
    sp = SamplingParams(max_tokens=8)
    eager = Executor(model, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=2, max_ctx=64, use_graphs=True)
    ex.capture_graphs()
    got = ex.generate_batch(prompts, sp)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert [r.output_ids for r in got] == [r.output_ids for r in eager]


def test_packed_linear_shards_are_block_bytes_of_the_full_matrix_cpu():
    """Row and column shards of a GGML-packed matrix are slices of its block bytes: the dequantised shard equals the
    same slice of the dequantised matrix; a column shard must be whole blocks."""
    from hibana_b200.models.bolt import GgmlLinear
    w = torch.randn(96, 256, generator=torch.Generator().manual_seed(0)) * 0.05
    lin = GgmlLinear.from_weight(w, name="x")
    full = lin.dequantize()
    rows = torch.tensor([5, 6, 7, 40, 41, 95])
    part = lin.shard(rows=rows, cols=slice(64, 192))
    assert isinstance(part, GgmlLinear) and (part.n, part.k) == (6, 128)
    assert torch.equal(part.dequantize(), full[rows][:, 64:192])
    assert torch.equal(lin.shard(rows=slice(32, 64)).dequantize(), full[32:64])
    with pytest.raises(ValueError):
        lin.shard(cols=slice(16, 80))
    x = torch.randn(3, 256, generator=torch.Generator().manual_seed(1)).bfloat16()
    y = lin(x).float()
    halves = lin.shard(cols=slice(0, 128))(x[:, :128].contiguous()).float() + lin.shard(cols=slice(128, 256))(x[:, 128:].contiguous()).float()
    assert (y - halves).abs().max() <= 2e-2 * y.abs().max() + 1e-3


def test_bolt_tensor_parallel_two_ranks_match_one_cpu():
    """The Bolt family under tensor parallelism: Q8_0 projections sharded as block bytes, IQ2 experts split by
    expert range with the block's all-reduce adding the ranks' partial sums. Two ranks (threads) emit the same tokens
    as each other and the first token of every request equals the unsharded model's."""
    import threading
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from test_tp import ThreadComm
    t = _small_bolt()
    full = HybridModel(t, "cpu", seed=0)
    shards = [HybridModel.sharded(t, 2, r, "cpu", seed=0) for r in range(2)]
    ffn_full = [b.ffn for b in full.blocks if b.ffn is not None]
    for r in range(2):
        ffns = [b.ffn for b in shards[r].blocks if b.ffn is not None]
        assert [f.experts.experts for f in ffns] == [3, 5, 3, 4] and all(f.partial for f in ffns)
        assert ffns[1].e_lo == 5 * r and ffns[1].experts.total == 10
        # this rank's experts are the block bytes of its range of the full stacks
        inter = ffn_full[1].experts.inter
        assert torch.equal(ffns[1].experts.fc1.raw, ffn_full[1].experts.fc1.raw[5 * r * inter:5 * (r + 1) * inter])
        assert ffns[0].shared.up.n == 128                           # the shared expert: half the columns each
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (20, 9)]
    sp = SamplingParams(max_tokens=4)
    ref = Executor(full, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)
    comm = ThreadComm(2)
    outs, errs = [None, None], []

    def run(rank):
        try:
            ex = Executor(shards[rank], max_batch=2, max_ctx=64, use_graphs=False, comm=comm.view(rank))
            outs[rank] = ex.generate_batch(prompts, sp)
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))
            comm.barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(180)
    assert not errs, errs
    a = [r.output_ids for r in outs[0]]
    assert a == [r.output_ids for r in outs[1]]
    assert sum(x[0] == y.output_ids[0] for x, y in zip(a, ref)) == len(a)


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,k", [(5, 2), (1100, 4)])
def test_packed_experts_by_range_partial_sums_add_up_on_gpu(tokens, k):
    """Experts split by range over two ranks (decode-sized: the GEMV skips pairs of the other range; prefill-sized:
    the grouped GEMMs take the range): the two partial sums add up to the whole layer's output."""
    e, h, inter = 8, 512, 256
    grid = _grid(256)
    fc1 = ops.random_blocks("iq2_xxs", e * inter, h, seed=25, scale=0.01)
    fc2 = ops.random_blocks("q8_0", e * h, inter, seed=26, scale=0.002)
    g = torch.Generator().manual_seed(27)
    x = torch.randn(tokens, h, generator=g).bfloat16().cuda()
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(tokens)]).int().cuda()
    wts = torch.rand(tokens, k, generator=g).cuda()
    whole = ops.PackedExperts(ops.PackedLinear(fc1.cuda(), "iq2_xxs", e * inter, h, grid),
                              ops.PackedLinear(fc2.cuda(), "q8_0", e * h, inter), e)
    want = whole.forward(x, ids, wts).float()
    parts = [whole.slice(r * 4, 4).forward(x, ids, wts, id_base=r * 4).float() for r in range(2)]
    torch.cuda.synchronize()
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0
    assert torch.isfinite(parts[0]).all() and torch.isfinite(parts[1]).all()
    assert (parts[0] + parts[1] - want).abs().max() <= 3e-2 * want.abs().max() + 1e-3
