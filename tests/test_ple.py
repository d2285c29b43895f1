import numpy as np
import pytest
import torch

from hibana_b200 import _native as nv
from hibana_b200.models.ple import PleTable, ngram_rows


@pytest.mark.skipif(not nv.LIB_PATH.exists(), reason="native library not built")
def test_row_gather_over_shards(tmp_path):
    rng = np.random.default_rng(0)
    row_bytes, per = 160, 1000
    shards, data = [], []
    for i in range(4):
        a = rng.integers(0, 256, size=(per, row_bytes), dtype=np.uint8)
        p = tmp_path / f"shard{i}.bin"
        a.tofile(p)
        shards.append(p)
        data.append(a)
    full = np.concatenate(data)
    t = PleTable(shards, row_bytes, per, threads=4)
    rows = rng.integers(0, 4 * per, size=(37, 5))
    got = t.gather(rows).numpy()
    assert got.shape == (37, 5, row_bytes) and np.array_equal(got, full[rows])
    with pytest.raises(IOError):
        t.gather(np.array([4 * per + 3]))
    t.close()
    res = PleTable(shards, row_bytes, per, resident_limit_bytes=1 << 30)
    assert np.array_equal(res.gather(rows).numpy(), full[rows])


def test_ngram_rows_are_causal_and_stable():
    ids = [5, 9, 9, 2, 7, 9, 9, 2]
    r = ngram_rows(ids, orders=(1, 2, 3), table_rows=1 << 20)
    assert r.shape == (8, 3)
    assert r[2, 0] == r[1, 0] == r[5, 0]           # unigram of token 9
    assert r[3, 1] == r[7, 1]                      # bigram (9, 2)
    assert r[3, 2] == r[7, 2]                      # trigram (9, 9, 2)
    assert np.array_equal(ngram_rows(ids[:5], (1, 2, 3), 1 << 20), r[:5])   # a prefix gives the same rows


def _naive_conv(x, weight, dilation, prev):
    """One sequence: rows [L, C], prev window [C, S] -> (conv [L, C], window after)."""
    k = weight.shape[1]
    s = (k - 1) * dilation
    full = torch.cat((prev.t().float(), x.float()), 0)             # [S + L, C]
    out = torch.zeros_like(x, dtype=torch.float32)
    for i in range(x.shape[0]):
        for j in range(k):
            out[i] += weight[:, j].float() * full[s + i - (k - 1 - j) * dilation]
    return out, full[-s:].t().to(prev.dtype)


def test_dilated_conv_over_ragged_sequences_matches_a_loop():
    from hibana_b200.models.ple import dilated_conv_ragged
    g = torch.Generator().manual_seed(0)
    c, k, d = 12, 4, 3
    s = (k - 1) * d
    weight = torch.randn(c, k, generator=g).to(torch.bfloat16)
    window = torch.randn(6, c, s, generator=g).to(torch.bfloat16)
    lens = [5, 1, 13, 2]
    x = torch.randn(sum(lens), c, generator=g).to(torch.bfloat16)
    ip = torch.tensor([0, 5, 6, 19, 21], dtype=torch.int32)
    slot_in = torch.tensor([2, 1, 4, 3])
    slot_out = torch.tensor([2, 5, 4, 0])
    has_init = torch.tensor([1, 1, 0, 1], dtype=torch.int32)
    before = window.clone()
    got = dilated_conv_ragged(x, weight, d, window, slot_in, slot_out, ip, has_init)
    for b, n in enumerate(lens):
        prev = before[slot_in[b]] * int(has_init[b])
        want, after = _naive_conv(x[ip[b]:ip[b + 1]], weight, d, prev)
        assert torch.allclose(got[ip[b]:ip[b + 1]].float(), want.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(window[slot_out[b]], after)
    # decode form: one row per sequence, no row pointers
    w2 = before.clone()
    xs = x[:3]
    got = dilated_conv_ragged(xs, weight, d, w2, torch.tensor([1, 2, 3]), torch.tensor([1, 2, 3]), None, None)
    for b in range(3):
        want, after = _naive_conv(xs[b:b + 1], weight, d, before[b + 1])
        assert torch.allclose(got[b].float(), want[0].to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(w2[b + 1], after)


def _flashnext_small(**kw):
    from hibana_b200.target import flashnext, scaled
    return scaled(flashnext(), layers=4, hidden=256, vocab=2048, q_heads=4, kv_heads=2, head_dim=64, gdn_k_heads=2,
                  gdn_v_heads=4, gdn_head_dim=64, experts=8, top_k=2, expert_ffn=128, shared_ffn=128, hyper_rank=32,
                  weight_format="bf16", kv_dtype="bf16", mtp_layers=1, mtp_depth=2, qsa_ratio=0, ple_rows=4096,
                  prefill_chunk=64, **kw)


def test_ple_layer_chunks_hash_and_history_cpu():
    """The layer's output for a sequence does not depend on how the sequence is cut into forwards (its window and
    token history carry over in the state pool), rows follow the 2- and 3-gram hashes, and an end-of-sequence token
    cuts the context."""
    from hibana_b200.cache.state_pool import StatePool
    from hibana_b200.engine.context import ForwardContext, PREFILL, DECODE
    from hibana_b200.models.layers import Init
    from hibana_b200.models.ple import PleLayer
    t = _flashnext_small()
    layer = PleLayer(t, Init(0, "cpu"), "ple")
    pool = StatePool(1, 4, 8, 4, (1, 1, 1), torch.device("cpu"))
    layer.register(pool)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(2, t.vocab, (11,), generator=g)
    hyper = torch.randn(11, t.hyper_streams * t.hidden, generator=g).to(torch.bfloat16)

    def ctx(mode, slots, ip=None, init=None):
        return ForwardContext(mode, positions=None, slots=None, kv_indices=None, ctx_len=None,
                              q_indptr=None if ip is None else torch.tensor(ip, dtype=torch.int32),
                              state_slots=torch.tensor(slots, dtype=torch.int32),
                              has_initial_state=None if init is None else torch.tensor(init, dtype=torch.int32))
    whole = layer.forward(hyper, ids, ctx(PREFILL, [1], [0, 11], [0]), pool)
    a = layer.forward(hyper[:7], ids[:7], ctx(PREFILL, [2], [0, 7], [0]), pool)
    b = layer.forward(hyper[7:10], ids[7:10], ctx(PREFILL, [2], [0, 3], [1]), pool)
    c = layer.forward(hyper[10:], ids[10:], ctx(DECODE, [2]), pool)
    assert torch.equal(torch.cat((a, b, c)), whole)
    assert torch.equal(pool.aux[layer.STATE_WINDOW][1], pool.aux[layer.STATE_WINDOW][2])
    assert pool.aux[layer.STATE_HISTORY][2].tolist() == ids[-2:].tolist()
    # hashes: same trailing n-gram, same rows; an end-of-sequence token hides what came before it
    eos = torch.tensor([t.ple_eos])
    r = layer.row_ids(torch.tensor([7, 7]), torch.tensor([5, 5]), torch.tensor([3, 9]))
    assert torch.equal(r[0, :layer.per], r[1, :layer.per]) and not torch.equal(r[0, layer.per:], r[1, layer.per:])
    cut = layer.row_ids(torch.tensor([7, 7]), eos.repeat(2), torch.tensor([3, 9]))
    assert torch.equal(cut[0], cut[1])
    assert int(r.min()) >= 0 and int(r.max()) < layer.rows.shape[0]
    pool.zero_slot(2)
    assert pool.aux[layer.STATE_HISTORY][2].tolist() == [t.ple_eos] * 2 and not pool.aux[layer.STATE_WINDOW][2].any()


def test_flashnext_with_ple_prefix_hits_and_speculation_cpu():
    """Flash-Next trunk with the per-layer embedding: prefix-cache hits (window and history restored from the
    snapshot), chunked prefill and MTP speculation (scratch slots + replay, as captured-round bodies) reproduce the
    plain run; the layer changes the tokens."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    t = _flashnext_small()
    m = HybridModel(t, "cpu", seed=0)
    assert 0 in m.ple
    g = torch.Generator().manual_seed(0)
    pre = torch.randint(2, t.vocab, (48,), generator=g).tolist()
    prompts = [pre + torch.randint(2, t.vocab, (16,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=10)

    def run(ex):
        outs = []
        for p in prompts:
            outs.append(ex.generate_batch([p], sp)[0].output_ids)
            ex.state.check()
        return outs
    ref = run(Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False))
    ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False)
    assert run(ex) == ref and ex.stats["cached_tokens"] > 0
    spec = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False)
    spec.enable_spec(2)
    assert run(spec) == ref and spec.spec.graphs.rounds > 0
    batch = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False).generate_batch(prompts, sp)
    assert [r.output_ids for r in batch] == ref
    from hibana_b200.target import scaled
    plain = HybridModel(scaled(t, ple_layers=()), "cpu", seed=0)
    other = Executor(plain, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False).generate_batch(prompts[:1], sp)
    assert other[0].output_ids != ref[0]


@pytest.mark.gpu
def test_ple_layer_and_flashnext_graphs_gpu():
    """The layer on the GPU equals the CPU layer; a Flash-Next stack at full width with it decodes the same tokens
    from CUDA graphs as eagerly, and its speculative rounds (draft graph, then verify + accept + replay of the
    recurrent layers, the window and the history in one graph) equal the eager rounds."""
    from hibana_b200 import _native as nv
    from hibana_b200.cache.state_pool import StatePool
    from hibana_b200.engine.context import ForwardContext, PREFILL
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.models.layers import Init
    from hibana_b200.models.ple import PleLayer
    from hibana_b200.target import flashnext, scaled
    t = scaled(flashnext(), layers=4, vocab=2048, experts=16, top_k=4, expert_ffn=128, shared_ffn=128, mtp_depth=2,
               qsa_ratio=0, ple_rows=4096)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(2, t.vocab, (21,), generator=g)
    hyper = torch.randn(21, t.hyper_streams * t.hidden, generator=g).to(torch.bfloat16)
    outs = []
    for dev in ("cpu", "cuda"):
        layer = PleLayer(t, Init(0, dev, "cpu"), "ple")
        pool = StatePool(1, 2, 8, 4, (1, 1, 1), torch.device(dev))
        layer.register(pool)
        ctx = ForwardContext(PREFILL, positions=None, slots=None, kv_indices=None, ctx_len=None,
                             q_indptr=torch.tensor([0, 13, 21], dtype=torch.int32, device=dev),
                             state_slots=torch.tensor([1, 2], dtype=torch.int32, device=dev),
                             has_initial_state=torch.tensor([0, 0], dtype=torch.int32, device=dev))
        outs.append((layer.forward(hyper.to(dev), ids.to(dev), ctx, pool).float().cpu(),
                     pool.aux[layer.STATE_WINDOW].float().cpu(), pool.aux[layer.STATE_HISTORY].cpu()))
    assert torch.allclose(outs[0][0], outs[1][0], atol=3e-2, rtol=3e-2)
    assert torch.allclose(outs[0][1], outs[1][1], atol=3e-2, rtol=3e-2) and torch.equal(outs[0][2], outs[1][2])
    m = HybridModel(t, "cuda", seed=0, init_device="cpu")
    assert 0 in m.ple
    prompts = [torch.randint(2, t.vocab, (n,), generator=g).tolist() for n in (40, 23)]
    sp = SamplingParams(max_tokens=12)
    eager = [r.output_ids for r in Executor(m, max_batch=2, max_ctx=128, use_graphs=False,
                                            radix_cache=False).generate_batch(prompts, sp)]
    ex = Executor(m, max_batch=2, max_ctx=128, use_graphs=True, radix_cache=False, buckets=(1, 2))
    ex.capture_graphs()
    assert [r.output_ids for r in ex.generate_batch(prompts, sp)] == eager
    spec_eager = Executor(m, max_batch=2, max_ctx=128, use_graphs=False, radix_cache=False, buckets=(1, 2))
    spec_eager.enable_spec(2)
    want = [r.output_ids for r in spec_eager.generate_batch(prompts, sp)]
    spec = Executor(m, max_batch=2, max_ctx=128, use_graphs=True, radix_cache=False, buckets=(1, 2))
    spec.enable_spec(2)
    spec.capture_graphs()
    assert [r.output_ids for r in spec.generate_batch(prompts, sp)] == want
    assert spec.spec.graphs.rounds > 0
    spec.state.check()
    torch.cuda.synchronize()
    assert nv.read_status() == 0
