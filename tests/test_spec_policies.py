"""Sampled acceptance (rejection sampling), relaxed greedy acceptance, depth policies, the n-gram proposer."""
import math

import pytest
import torch

from hibana_b200.engine import depth as dp
from hibana_b200.engine import rejection as rj
from hibana_b200.engine.contracts import Capabilities, ProposerRequirements, check_capabilities
from hibana_b200.proposers import make_proposer


def test_distribution_truncation():
    lg = torch.tensor([[2.0, 1.0, 0.0, -1.0], [0.0, 0.0, 5.0, 0.0]])
    d = rj.distribution(lg, temperature=1.0, top_k=2)
    assert torch.count_nonzero(d[0]) == 2 and abs(float(d[0].sum()) - 1) < 1e-6
    d = rj.distribution(lg, temperature=torch.tensor([1.0, 0.0]), top_k=0, top_p=torch.tensor([0.7, 1.0]))
    assert torch.count_nonzero(d[0]) == 2          # 0.64 + the token that crosses 0.7
    assert d[1].tolist() == [0, 0, 1, 0]           # temperature 0 = argmax


def test_batch_matches_row_rule():
    g = torch.Generator().manual_seed(0)
    b, k, v = 64, 4, 50
    p = rj.distribution(torch.randn(b * (k + 1), v, generator=g) * 2, 0.9, 20, 0.95).view(b, k + 1, v)
    q = rj.distribution(torch.randn(b * k, v, generator=g) * 2, 1.0).view(b, k, v)
    drafts = torch.multinomial(q.view(-1, v), 1, generator=g).view(b, k)
    u = torch.rand(b, k + 1, generator=g)
    ru = torch.rand(b, k + 1, generator=g)
    for soft in (0.0, 0.5):
        ver = rj.verify_batch(p, q, drafts, u, ru, soft=soft)
        for i in range(b):
            em, acc = rj.verify_row(list(p[i]), list(q[i]), drafts[i].tolist(), u[i].tolist(), ru[i].tolist(), soft)
            assert int(ver.accepted[i]) == acc and ver.emitted[i, :acc + 1].tolist() == em
    # slack can only accept more
    assert int(rj.verify_batch(p, q, drafts, u, ru, 0.5).accepted.sum()) >= int(rj.verify_batch(p, q, drafts, u, ru).accepted.sum())


def test_speculative_sampling_preserves_the_target_law():
    """First emitted token ~ p_0 whatever the draft law is (the defining property)."""
    g = torch.Generator().manual_seed(1)
    v, n = 6, 40000
    p0 = torch.tensor([0.4, 0.25, 0.15, 0.1, 0.07, 0.03])
    q1 = torch.tensor([0.05, 0.05, 0.3, 0.3, 0.2, 0.1])
    p = torch.stack([p0, torch.full((v,), 1 / v)]).expand(n, 2, v).contiguous()
    q = q1.expand(n, 1, v).contiguous()
    drafts = torch.multinomial(q1, n, replacement=True, generator=g).view(n, 1)
    ver = rj.verify_batch(p, q, drafts, torch.rand(n, 2, generator=g), torch.rand(n, 2, generator=g))
    freq = torch.bincount(ver.emitted[:, 0], minlength=v).float() / n
    assert float((freq - p0).abs().max()) < 0.012
    assert 0.3 < float(ver.accepted.float().mean()) < 0.7      # sum min(p, q) = 0.5


def test_relaxed_greedy():
    rank = torch.tensor([[0, 1, 3], [2, 0, 1]])
    gap = torch.tensor([[0.0, 0.4, 0.1], [0.2, 0.0, 2.0]])
    got = rj.relaxed_greedy(rank, gap, top_k=3, margin=0.5)
    assert got.tolist() == [[True, True, False], [True, True, False]]
    assert rj.relaxed_greedy(rank, gap, top_k=1, margin=0.0).tolist() == [[True, False, False], [False, True, False]]


class _Req:
    def __init__(self, rid, ids=()):
        self.rid, self.all_ids = rid, list(ids)


def test_depth_policies():
    assert dp.parse_depths("8:4, 1:6,32:2") == [(1, 6), (8, 4), (32, 2)]
    with pytest.raises(ValueError):
        dp.parse_depths("4")
    bd = dp.BatchDepth("1:6,8:4,32:0")
    assert [bd.depth_for(n) for n in (1, 7, 8, 31, 32, 200)] == [6, 6, 4, 4, 0, 0]
    ad = dp.AcceptanceDepth(max_depth=8, row_cost=0.3)
    r = _Req(1)
    d0 = ad.depth_for(r)
    for _ in range(40):
        ad.observe(r, 4, 0)                      # always rejected at the first position
    low = ad.depth_for(r)
    for _ in range(80):
        ad.observe(r, 4, 4)
    high = ad.depth_for(r)
    assert low < d0 < high <= 8 and low >= 1
    assert abs(dp.expected_tokens(0.5, 3) - 1.875) < 1e-9
    rb = dp.RowBudget(rows=8)
    kept = rb.choose([[0.9, 0.9, 0.9, 0.9], [0.5, 0.1, 0.1, 0.1], [0.95, 0.2, 0.9, 0.9]])
    assert sum(kept) == 8 - 3 and kept == [4, 0, 1]      # 0.9^4 = 0.656 still beats 0.5
    assert dp.ragged_budgets(4, 16, 8) == 3


def test_ngram_proposer_and_capabilities():
    pr = make_proposer("ngram")
    seq = [5, 6, 7, 8, 9, 1, 2, 5, 6, 7]
    out = pr.propose([_Req(1, seq), _Req(2, [1, 2, 3])], 3)
    assert out.tokens[0].tolist() == [8, 9, 1] and out.lengths == [3, 0]
    assert float(out.scores[1].sum()) == 0.0
    check_capabilities(pr.capabilities, ProposerRequirements(row_budget=True, depth=8))
    with pytest.raises(ValueError):
        check_capabilities(Capabilities(max_depth=4), ProposerRequirements(depth=6, row_budget=True))
    with pytest.raises(ValueError):
        make_proposer("nope")


def test_ngram_proposer_in_the_engine_is_exact_cpu():
    """Any proposer plugs into the speculative round: n-gram drafts are verified by the target, so the output equals
    plain greedy decoding token for token, and repeated text gets several tokens per round."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, t.vocab, (12,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, t.vocab, (20,), generator=g).tolist()]
    sp = SamplingParams(max_tokens=16)
    plain = Executor(model, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex.enable_spec(depth=4, proposer="ngram")
    spec = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in spec] == [r.output_ids for r in plain]
    assert ex.spec.stats.rounds > 0 and ex.spec.stats.emitted >= ex.spec.stats.rounds


def test_block_drafter_lattice_and_engine_exactness_cpu():
    """Block drafter: one forward gives a candidate lattice; greedy / sampled walks agree with their definitions;
    through the engine the output equals plain decoding (greedy) whatever the random drafter proposes."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.models.parallel_draft import greedy_lattice, sample_lattice
    from hibana_b200.target import dense_tiny, scaled
    g = torch.Generator().manual_seed(0)
    cand = torch.randint(0, 50, (2, 3, 4), generator=g)
    scores = torch.randn(2, 3, 4, 4, generator=g)
    toks, idx = greedy_lattice(cand, scores)
    for b in range(2):
        prev = 0
        for j in range(3):
            prev = int(scores[b, j, prev].argmax())
            assert int(idx[b, j]) == prev and int(toks[b, j]) == int(cand[b, j, prev])
    u = torch.rand(2, 3, generator=g)
    st, laws = sample_lattice(cand, scores, torch.tensor([1.0, 0.7]), u, 50)
    assert laws.shape == (2, 3, 50) and torch.allclose(laws.sum(-1), torch.ones(2, 3), atol=1e-5)
    assert (laws.gather(2, st[..., None]) > 0).all()
    # the one-launch walk (ops/sampling.py) makes the same choices and reports the same laws on the candidates
    from hibana_b200.ops import sampling
    wt, wi, wp, we = sampling.lattice_walk(cand, scores)
    assert torch.equal(wt, toks) and torch.equal(wi.long(), idx)
    wt, wi, wp, we = sampling.lattice_walk(cand, scores, torch.tensor([1.0, 0.7]), u)
    assert torch.equal(wt, st)
    dense = torch.zeros(2, 3, 50).scatter_add_(2, cand, wp)
    assert torch.allclose(dense, laws, atol=1e-6) and bool(((we > 0) & (we <= 1)).all())
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (19, 33)]
    sp = SamplingParams(max_tokens=12)
    plain = Executor(model, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex.enable_spec(depth=5, proposer=make_proposer("dflash2", executor=ex, layers=1, heads=4, window=32))
    spec = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in spec] == [r.output_ids for r in plain]
    assert ex.spec.stats.rounds > 0
    # sampled requests: drafts come with their laws and the round still terminates with valid tokens
    ex2 = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex2.enable_spec(depth=3, proposer=make_proposer("dflash2", executor=ex2, layers=1, heads=4, window=32))
    out = ex2.generate_batch(prompts, SamplingParams(max_tokens=8, temperature=0.8, seed=11))
    assert all(len(r.output_ids) == 8 and all(0 <= x < t.vocab for x in r.output_ids) for r in out)


@pytest.mark.gpu
def test_block_drafter_on_gpu_is_exact():
    """The block drafter runs on the device (bf16 weights, shared embedding / head of the target); greedy output with
    it equals plain greedy decoding on the same GPU model."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cuda", seed=0, init_device="cpu")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (40, 70)]
    sp = SamplingParams(max_tokens=16)
    plain = Executor(model, max_batch=4, max_ctx=160, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=160, use_graphs=False)
    ex.enable_spec(depth=5, proposer=make_proposer("dflash2", executor=ex, layers=1, heads=4, window=64))
    spec = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in spec] == [r.output_ids for r in plain]
    assert ex.spec.stats.rounds > 0


def test_device_rounds_equal_host_rounds_cpu():
    """The captured-round form (static buffers, verify + accept kernel in one body, one META readback) makes the
    same decisions as the host round: same tokens, same tokens per round, stop ids and budgets honoured, padded
    bucket rows harmless; and it moves one upload and one readback per round."""
    import torch
    from hibana_b200 import config as cfgmod
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(8)
    base = torch.randint(0, t.vocab, (10,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, t.vocab, (18,), generator=g).tolist(), base * 2 + base[:4]]
    plain = Executor(model, max_batch=4, max_ctx=160, use_graphs=False).generate_batch(
        prompts, SamplingParams(max_tokens=20))
    stop_tok = plain[0].output_ids[7]
    params = [SamplingParams(max_tokens=20, stop_ids=(stop_tok,)), SamplingParams(max_tokens=11),
              SamplingParams(max_tokens=20)]
    outs = {}
    for on in (False, True):
        with cfgmod.using(device_accept=on):
            ex = Executor(model, max_batch=4, max_ctx=160, use_graphs=False, buckets=(1, 4))
            ex.enable_spec(depth=3, proposer="ngram")
            assert (ex.spec.graphs is not None) == on
            res = ex.generate_batch(prompts, params)
            outs[on] = ([r.output_ids for r in res], [r.rounds for r in res], [r.finish_reason for r in res],
                        ex.spec.graphs.rounds if on else 0)
    assert outs[True][:3] == outs[False][:3]
    assert outs[True][3] > 0
    assert outs[True][0][0][-1] == stop_tok and outs[True][2][0] == "stop"
    assert len(outs[True][0][1]) == 11 and outs[True][2][1] == "length"
    ref = [r.output_ids for r in plain]
    assert outs[True][0][2] == ref[2] and outs[True][0][1] == ref[1][:11]
    # sampled requests (and a greedy one beside them) take the same device round: the rejection-sampling rule is
    # the kernel-shaped `spec_targets` in both, so tokens, rounds and the draw counters agree
    params = [SamplingParams(max_tokens=16, temperature=0.8, top_k=50, top_p=0.9, seed=5), SamplingParams(max_tokens=12),
              SamplingParams(max_tokens=16, temperature=1.1, seed=9)]
    outs = {}
    for on in (False, True):
        with cfgmod.using(device_accept=on):
            ex = Executor(model, max_batch=4, max_ctx=160, use_graphs=False, buckets=(1, 4))
            ex.enable_spec(depth=3, proposer="ngram")
            res = ex.generate_batch(prompts, params)
            outs[on] = ([r.output_ids for r in res], [r.rounds for r in res], [r.draws for r in res],
                        ex.spec.graphs.rounds if on else 0)
    assert outs[True][:3] == outs[False][:3] and outs[True][3] > 0
    assert outs[True][0][1] == ref[1][:12]                       # the greedy request is unaffected by its neighbours


@pytest.mark.gpu
def test_captured_verify_rounds_on_gpu_are_exact():
    """CUDA-graph verify + device accept: the n-gram speculative engine equals plain greedy decoding token for
    token on the GPU, with the rounds running as graph replays (one upload, one readback each)."""
    import torch
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny
    t = dense_tiny()
    model = DenseModel(t, "cuda:0", seed=0)
    g = torch.Generator().manual_seed(8)
    base = torch.randint(0, t.vocab, (10,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, t.vocab, (18,), generator=g).tolist(), base * 2 + base[:4]]
    sp = SamplingParams(max_tokens=24)
    plain = Executor(model, max_batch=4, max_ctx=256, use_graphs=True)
    plain.capture_graphs()
    want = [r.output_ids for r in plain.generate_batch(prompts, sp)]
    ex = Executor(model, max_batch=4, max_ctx=256, use_graphs=True, buckets=(1, 2, 4))
    ex.enable_spec(depth=2, proposer="ngram")
    ex.capture_graphs()
    assert ex.spec.graphs is not None and all(b.graph is not None for b in ex.spec.graphs.bufs.values())
    h2d0, d2h0 = ex.runner.h2d_bytes, ex.runner.d2h_bytes
    got = ex.generate_batch(prompts, sp)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert [r.output_ids for r in got] == want
    assert ex.spec.graphs.rounds > 0 and ex.spec.stats.emitted >= ex.spec.stats.rounds
    # sampled requests replay the same graphs (the sampled-verify kernel sits after the head inside them) and are
    # reproducible from their seeds
    sp2 = [SamplingParams(max_tokens=20, temperature=0.9, top_p=0.9, seed=3), SamplingParams(max_tokens=20),
           SamplingParams(max_tokens=20, temperature=0.7, top_k=40, seed=4)]
    rounds0 = ex.spec.graphs.rounds
    a = [r.output_ids for r in ex.generate_batch(prompts, sp2)]
    b = [r.output_ids for r in ex.generate_batch(prompts, sp2)]
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert a == b and a[1] == want[1][:20] and ex.spec.graphs.rounds > rounds0
    assert a[0] != want[0][:20] or a[2] != want[2][:20]         # temperature did something


def test_draft_heads_shortlist_and_vocab_parallel_cpu():
    """Draft heads: a row subset scores only its rows, a 3-bit copy with rescoring picks the full head's argmax
    whenever it is shortlisted, and the vocabulary-parallel head (two ranks played by two threads) returns the
    candidates of the unsharded head on both ranks."""
    import threading
    import torch
    from hibana_b200.proposers import draft_head as dh
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_tp import ThreadComm
    g = torch.Generator().manual_seed(0)
    head = (torch.randn(512, 128, generator=g) * 0.5).bfloat16()
    x = torch.randn(9, 128, generator=g).bfloat16()
    full = (x.float() @ head.float().t())
    t = dh.TargetHead(lambda h: h.float() @ head.float().t())
    assert torch.equal(t.argmax(x), full.argmax(-1))
    ids, vals = t.candidates(x, 3)
    assert torch.equal(ids, full.topk(3, -1).indices) and t.bytes == 0
    sub = torch.arange(0, 512, 2)
    s = dh.ShortlistHead(head, sub)
    assert torch.equal(s.argmax(x), sub[full[:, ::2].argmax(-1)]) and s.bytes == 256 * 128 * 2
    w3 = dh.ShortlistHead(head, None, "w3", rescore=8)
    agree = (w3.argmax(x) == full.argmax(-1)).float().mean()
    assert agree >= 0.85 and w3.bytes < head.numel() * 2 / 3
    c_ids, c_vals = w3.candidates(x, 4)
    assert c_ids.shape == (9, 4) and bool((c_vals[:, :-1] >= c_vals[:, 1:]).all())
    conf = t.argmax_confidence(x)[1]
    assert conf.shape == (9, 2) and bool((conf[:, 0] >= conf[:, 1]).all())
    comm = ThreadComm(2)
    outs = [None, None]

    def run(rank):
        vp = dh.VocabParallelHead(head[rank * 256:(rank + 1) * 256].contiguous(), comm.view(rank), rank)
        outs[rank] = (vp.candidates(x, 3), vp.argmax(x), vp.argmax_confidence(x)[1])
    th = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for a in th:
        a.start()
    for a in th:
        a.join(30)
    for r in range(2):
        (ids_r, vals_r), am, cf = outs[r]
        assert torch.equal(ids_r, full.topk(3, -1).indices) and torch.equal(am, full.argmax(-1))
        assert torch.allclose(vals_r, full.topk(3, -1).values, atol=1e-4)
        assert torch.allclose(cf, conf, atol=1e-4)


def _attn_mtp_model(device):
    """Attention-only hybrid with an MTP head (no recurrent state: the whole round can stay on the device)."""
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import ATTN, MLP, Target
    t = Target(name="attn-mtp", family="hybrid_moe", hidden=256, vocab=2048, layers=((ATTN, MLP),) * 2, q_heads=4,
               kv_heads=2, head_dim=64, rope_theta=1e4, ffn=512, mtp_layers=1, mtp_depth=3, max_context=512,
               prefill_chunk=128)
    return HybridModel(t, device, seed=0)


def test_mtp_round_with_draft_graphs_equals_plain_decoding_cpu():
    """MTP drafting as one chained body per bucket, the drafts handed to the verify body without a host copy:
    the engine still emits exactly the plain greedy tokens, and sampled requests are reproducible."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    model = _attn_mtp_model("cpu")
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (21, 33, 9)]
    sp = SamplingParams(max_tokens=14, ignore_eos=True)
    want = [r.output_ids for r in Executor(model, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)]
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False, buckets=(1, 4))
    ex.enable_spec(depth=3)
    assert ex.spec.draft_graphs is not None
    got = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in got] == want
    assert ex.spec.draft_graphs.rounds > 0 and ex.spec.graphs.rounds == ex.spec.draft_graphs.rounds
    sampled = [SamplingParams(max_tokens=10, temperature=0.9, seed=s, ignore_eos=True) for s in (1, 2, 3)]
    a = [r.output_ids for r in ex.generate_batch(prompts, sampled)]
    b = [r.output_ids for r in ex.generate_batch(prompts, sampled)]
    assert a == b


@pytest.mark.gpu
def test_mtp_round_graphs_on_gpu():
    """Draft graph + verify graph per round on the GPU: tokens equal plain greedy decoding."""
    import torch
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    model = _attn_mtp_model("cuda:0")
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (21, 33, 9)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    plain = Executor(model, max_batch=4, max_ctx=256, use_graphs=True)
    plain.capture_graphs()
    want = [r.output_ids for r in plain.generate_batch(prompts, sp)]
    ex = Executor(model, max_batch=4, max_ctx=256, use_graphs=True, buckets=(1, 4))
    ex.enable_spec(depth=3)
    ex.capture_graphs()
    assert all(b.graph is not None for b in ex.spec.draft_graphs.bufs.values())
    got = ex.generate_batch(prompts, sp)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert [r.output_ids for r in got] == want
    assert ex.spec.draft_graphs.rounds > 0 and ex.spec.stats.emitted >= ex.spec.stats.rounds


def test_lilicorr_drafter_conv_correlator_and_engine_exactness_cpu():
    """LiLiCorr: the two-tap convolution is causal over block positions, the correlator gives a [k, W, W] lattice
    whose first slot does not depend on a previous choice, and the engine with it as proposer emits plain greedy
    tokens."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.models.lilicorr import LiLiCorrDrafter, two_tap_conv
    from hibana_b200.target import dense_tiny, scaled
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 5, 64, generator=g)
    coeff = torch.randn(2, 5, 2, 4, generator=g) * 0.1
    base = torch.randn(2, 64, generator=g)
    y = two_tap_conv(x, coeff, base)
    x2 = x.clone()
    x2[:, 3] += 1.0                                              # position 3 reaches positions 3 and 4 only
    d = (two_tap_conv(x2, coeff, base) - y).abs().amax(-1)
    assert bool((d[:, :3] == 0).all()) and bool((d[:, 3:] > 0).all())
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    dr = LiLiCorrDrafter(t.hidden, t.vocab, model.embed, model.lm_head, topk=4, layers=1, heads=4, window=64)
    hidden = torch.randn(3, 5, t.hidden, generator=g)
    dr._anchor_feat = torch.randn(3, t.hidden, generator=g)
    cand, scores = dr.select(hidden, torch.tensor([1, 2, 3]))
    assert cand.shape == (3, 5, 4) and scores.shape == (3, 5, 4, 4)
    assert torch.allclose(scores[:, 0, 0], scores[:, 0, 3])      # slot 0: the same row for every "previous choice"
    assert not torch.allclose(scores[:, 1, 0], scores[:, 1, 3])
    prompts = [torch.randint(0, t.vocab, (n,), generator=g).tolist() for n in (19, 33)]
    sp = SamplingParams(max_tokens=12)
    plain = Executor(model, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex.enable_spec(depth=4, proposer="lilicorr")
    got = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in got] == [r.output_ids for r in plain]
    assert ex.spec.stats.rounds > 0
