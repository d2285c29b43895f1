"""Hybrid model families end to end: prefix-cache hits with recurrent snapshots, MTP speculation == plain greedy,
GPU kernels vs the CPU path."""
import pytest
import torch

from hibana_b200.engine.executor import Executor
from hibana_b200.engine.request import SamplingParams
from hibana_b200.models.hybrid import HybridModel
from hibana_b200.target import flashnext, nemotron, qwen38_hybrid, scaled, tiny_hybrid_moe


def _workload(t, n=4, shared=48, tail=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    pre = torch.randint(0, t.vocab, (shared,), generator=g).tolist()
    return [pre + torch.randint(0, t.vocab, (tail,), generator=g).tolist() for _ in range(n)]


def _run(ex, prompts, n=8):
    outs = []
    for p in prompts:
        outs.append(ex.generate_batch([p], SamplingParams(max_tokens=n))[0].output_ids)
        ex.state.check()
    return outs


def test_tiny_hybrid_prefix_hits_match_cold_cpu():
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=0)
    prompts = _workload(t)
    ref = _run(Executor(m, max_batch=4, max_ctx=128, use_graphs=False, radix_cache=False), prompts)
    ex = Executor(m, max_batch=4, max_ctx=128, use_graphs=False)
    assert _run(ex, prompts) == ref
    assert ex.stats["cached_tokens"] == 96          # requests 3 and 4 resume from the 48-token snapshot
    assert ex.state.cache.full_reprefills == 1      # request 2 found KV but no snapshot


def test_mtp_speculation_equals_plain_greedy_cpu():
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=0)
    prompts = _workload(t, n=3)
    ref = _run(Executor(m, max_batch=4, max_ctx=160, use_graphs=False), prompts, n=32)
    ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False)
    ex.enable_spec(2)
    got = _run(ex, prompts, n=32)
    assert got == ref
    s = ex.spec.stats.as_dict()
    assert s["rounds"] > 0 and 1.0 <= s["tokens_per_round"] <= 3.0
    ex.state.cache.flush()
    assert ex.kv.free_count == ex.kv.slots


def test_captured_rounds_replay_recurrent_state_cpu():
    """A model with recurrent layers takes the captured-round form too: the verify body writes its end state to
    scratch slots, logs the recurrent inputs, and replays the accepted rows from the device-side counts. Tokens,
    tokens per round and finish reasons equal the host round's; the MTP chain runs as its drafting body; the
    scratch slots are accounted for in the pool's ledger."""
    from hibana_b200 import config as cfgmod
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=0)
    prompts = _workload(t, n=3, seed=5)
    params = [SamplingParams(max_tokens=18), SamplingParams(max_tokens=9),
              SamplingParams(max_tokens=14, temperature=0.8, top_p=0.9, seed=7)]
    outs = {}
    for on in (False, True):
        with cfgmod.using(device_accept=on):
            ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False, buckets=(1, 4))
            ex.enable_spec(2)
            res = ex.generate_batch(prompts, params)
            ex.state.check()
            outs[on] = ([r.output_ids for r in res], [r.rounds for r in res], [r.finish_reason for r in res])
            if on:
                assert ex.spec.graphs.rounds > 0 and ex.spec.draft_graphs.rounds == ex.spec.graphs.rounds
                assert ex.state_pool.reserved == 4 and not ex.spec.scratch
    assert outs[True] == outs[False]
    ref = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False).generate_batch(prompts, params[:2])
    assert outs[True][0][:2] == [r.output_ids for r in ref]


def test_batched_speculation_with_stop_and_budget_cpu():
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=1)
    prompts = _workload(t, n=3, seed=3)
    plain = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False)
    ref = plain.generate_batch(prompts, SamplingParams(max_tokens=11))
    stop = ref[0].output_ids[5]
    ref2 = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False).generate_batch(
        prompts, SamplingParams(max_tokens=11, stop_ids=(stop,)))
    ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False)
    ex.enable_spec(3)
    got = ex.generate_batch(prompts, SamplingParams(max_tokens=11, stop_ids=(stop,)))
    for a, b in zip(got, ref2):
        assert a.finish_reason == b.finish_reason and len(a.output_ids) == len(b.output_ids)
        assert a.output_ids[0] == b.output_ids[0]
    ex.state.check()


@pytest.mark.parametrize("make", [qwen38_hybrid, flashnext, nemotron])
def test_reference_families_run_scaled_cpu(make):
    t = make()
    small = dict(hidden=256, vocab=512, q_heads=4, kv_heads=2, head_dim=64, ffn=256 if t.ffn else 0,
                 gdn_k_heads=2 if t.gdn_k_heads else 0, gdn_v_heads=4 if t.gdn_v_heads else 0,
                 gdn_head_dim=32, mamba_heads=8 if t.mamba_heads else 0, mamba_head_dim=32, mamba_state=16,
                 mamba_groups=2 if t.mamba_heads else 1, experts=8 if t.experts else 0,
                 top_k=min(t.top_k, 3), expert_ffn=128 if t.experts else 0, shared_ffn=128 if t.shared_ffn else 0,
                 latent=128 if t.latent else 0, weight_format="bf16", kv_dtype="bf16", mtp_layers=0,
                 max_context=512)
    layers = t.layers[:8] if t.family != "nemotron" else t.layers[:9]
    st = scaled(t, **small)
    st = scaled(st, layers=None) if False else st
    import dataclasses
    st = dataclasses.replace(st, layers=layers)
    m = HybridModel(st, "cpu", seed=0)
    ex = Executor(m, max_batch=2, max_ctx=96, use_graphs=False)
    out = ex.generate_batch(_workload(st, n=2, shared=20, tail=6), SamplingParams(max_tokens=4))
    assert all(len(r.output_ids) == 4 for r in out)
    ex.state.check()


@pytest.mark.gpu
def test_tiny_hybrid_gpu_matches_cpu_and_graphs():
    t = tiny_hybrid_moe()
    cpu = HybridModel(t, "cpu", seed=0)
    gpu = HybridModel(t, "cuda", seed=0, init_device="cpu")
    prompts = _workload(t)
    ref = _run(Executor(cpu, max_batch=4, max_ctx=128, use_graphs=False), prompts, n=16)
    ex = Executor(gpu, max_batch=4, max_ctx=128, use_graphs=True)
    ex.capture_graphs()
    got = _run(ex, prompts, n=16)
    assert [g[0] for g in got] == [r[0] for r in ref]
    same = sum(a == b for x, y in zip(got, ref) for a, b in zip(x, y))
    assert same >= 0.6 * 64
    assert ex.stats["cached_tokens"] == 96
    eager = _run(Executor(gpu, max_batch=4, max_ctx=128, use_graphs=False), prompts, n=16)
    assert eager == got                                    # graph replay == eager
    ex2 = Executor(gpu, max_batch=4, max_ctx=160, use_graphs=False)
    ex2.enable_spec(2)
    spec = _run(ex2, prompts, n=16)
    agree = sum(a == b for x, y in zip(spec, eager) for a, b in zip(x, y))
    assert [s[0] for s in spec] == [e[0] for e in eager] and agree >= 0.7 * 64
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0
    # the same rounds as CUDA graphs: MTP chain graph, then verify + accept + recurrent replay in one graph
    ex3 = Executor(gpu, max_batch=4, max_ctx=160, use_graphs=True, buckets=(1, 4))
    ex3.enable_spec(2)
    ex3.capture_graphs()
    assert all(b.graph is not None for b in ex3.spec.graphs.bufs.values())
    assert _run(ex3, prompts, n=16) == spec
    assert ex3.spec.graphs.rounds > 0 and ex3.spec.draft_graphs.rounds == ex3.spec.graphs.rounds
    batch = ex3.generate_batch(prompts[:3], SamplingParams(max_tokens=12))
    ex3.state.check()
    assert [r.output_ids[0] for r in batch] == [s[0] for s in spec[:3]]
    torch.cuda.synchronize()
    assert nv.read_status() == 0


def test_relaxed_and_sampled_acceptance_cpu():
    """Relaxed greedy accepts at least as many drafts as exact greedy; sampled requests run through speculative
    sampling, reproducibly for a fixed seed, and keep every bookkeeping invariant."""
    t = tiny_hybrid_moe()
    m = HybridModel(t, "cpu", seed=0)
    prompts = _workload(t, n=3)

    def run(params):
        ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False)
        ex.enable_spec(2)
        out = [r.output_ids for r in ex.generate_batch(prompts, params)]
        ex.state.check()
        st = ex.spec.stats.as_dict()
        ex.state.cache.flush()
        assert ex.kv.free_count == ex.kv.slots
        return out, st

    exact, s_exact = run(SamplingParams(max_tokens=24))
    relaxed, s_rel = run(SamplingParams(max_tokens=24, accept_top_k=4, accept_margin=50.0))
    assert s_rel["accepted"] >= s_exact["accepted"] and s_rel["tokens_per_round"] >= s_exact["tokens_per_round"]
    assert [r[0] for r in relaxed] == [r[0] for r in exact] and all(len(r) == 24 for r in relaxed)
    a, s_a = run(SamplingParams(max_tokens=24, temperature=0.8, top_k=20, top_p=0.95, seed=7))
    b, _ = run(SamplingParams(max_tokens=24, temperature=0.8, top_k=20, top_p=0.95, seed=7))
    c, _ = run(SamplingParams(max_tokens=24, temperature=0.8, top_k=20, top_p=0.95, seed=8))
    assert a == b and a != c and all(len(r) == 24 for r in a)
    assert s_a["rounds"] > 0 and all(0 <= tok < t.vocab for r in a for tok in r)


def test_hyper_connections_in_the_trunk_cpu():
    """With hyper_streams > 1 the trunk carries several residual streams per token (models/hyper.py sites around every
    sublayer). Prefix-cache hits, chunked prefill and MTP speculation must still reproduce the plain run."""
    t = scaled(tiny_hybrid_moe(), hyper_streams=2, hyper_rank=16)
    m = HybridModel(t, "cpu", seed=0)
    assert m.hyper_sites is not None and len(m.hyper_sites) == 2 * len(t.layers) + 1
    prompts = _workload(t, n=3)
    ref = _run(Executor(m, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False), prompts, n=12)
    ex = Executor(m, max_batch=4, max_ctx=160, use_graphs=False)
    ex.enable_spec(2)
    assert _run(ex, prompts, n=12) == ref
    plain = HybridModel(scaled(tiny_hybrid_moe()), "cpu", seed=0)
    other = _run(Executor(plain, max_batch=4, max_ctx=160, use_graphs=False, radix_cache=False), prompts[:1], n=12)
    assert other != ref[:1]                      # the hyper trunk is a different function of the same seed


def _w3_model(device):
    t = scaled(tiny_hybrid_moe(), expert_ffn=128, mtp_layers=0, mtp_depth=0)
    m = HybridModel(t, device, seed=0, init_device="cpu")
    added = m.attach_w3()
    return t, m, added


def test_hybrid_w3_copies_cover_projections_and_experts_cpu():
    """`attach_w3` on a hybrid: every tiled projection and every MoE layer's routed experts get a 3-bit decode copy;
    decode-sized calls run on the copies (prefill chunks above the row limit keep the served weights) and the step's
    logits stay close to the served model's."""
    from hibana_b200.models.layers import MoeLayer
    from hibana_b200.models.linear import W3_MAX_ROWS
    t, m, added = _w3_model("cpu")
    ref = HybridModel(t, "cpu", seed=0)
    moes = [b.ffn for b in m.blocks if isinstance(b.ffn, MoeLayer)]
    assert moes and all(f.experts_w3 is not None and f.experts_w3.fmt == "w3" for f in moes)
    assert added > 0 and all(lin.w3 is not None for lin in m.linears() if not lin.name.endswith(".router"))
    assert moes[0].router.w3 is None
    x = torch.randn(3, t.hidden).bfloat16()
    assert moes[0]._ew(x) is moes[0].experts_w3
    assert moes[0]._ew(torch.zeros(W3_MAX_ROWS + 1, t.hidden)) is moes[0].experts
    # one MoE layer: 3-bit experts against the served ones
    a, b = moes[0].forward(x).float(), [bb.ffn for bb in ref.blocks if isinstance(bb.ffn, MoeLayer)][0].forward(x).float()
    assert (a - b).norm() <= 0.35 * b.norm()
    prompts = _workload(t, n=2)
    sp = SamplingParams(max_tokens=4)
    got = Executor(m, max_batch=2, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    assert all(len(r.output_ids) == 4 for r in got)


@pytest.mark.gpu
def test_hybrid_w3_copies_decode_on_gpu_matches_cpu_copies():
    """The same 3-bit copies on the GPU (dequantisation fused into the plain and the grouped GEMM): a decode-sized
    MoE layer call and a trunk forward agree with the CPU evaluation of the same copies."""
    from hibana_b200 import _native as nv
    from hibana_b200.models.layers import MoeLayer
    t, cpu, _ = _w3_model("cpu")
    _, gpu, _ = _w3_model("cuda")
    x = torch.randn(5, t.hidden, generator=torch.Generator().manual_seed(3)).bfloat16()
    fc = [b.ffn for b in cpu.blocks if isinstance(b.ffn, MoeLayer)][0]
    fg = [b.ffn for b in gpu.blocks if isinstance(b.ffn, MoeLayer)][0]
    a, b = fc.forward(x).float(), fg.forward(x.cuda()).float().cpu()
    assert (a - b).abs().max() <= 3e-2 * a.abs().max() + 1e-3
    prompts = _workload(t, n=2)
    sp = SamplingParams(max_tokens=6)
    want = Executor(cpu, max_batch=2, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(gpu, max_batch=2, max_ctx=128, use_graphs=True)
    ex.capture_graphs()
    got = ex.generate_batch(prompts, sp)
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert [r.output_ids[0] for r in got] == [r.output_ids[0] for r in want]
