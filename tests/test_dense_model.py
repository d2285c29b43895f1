"""Dense decoder end to end through the Executor: CPU self-consistency and GPU-vs-CPU agreement."""
import pytest
import torch

from hibana_b200.engine.executor import Executor
from hibana_b200.engine.request import SamplingParams
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled


def _prompts(n, length, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def test_chunked_prefill_matches_single_pass_cpu():
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    prompts = _prompts(3, 21, t.vocab)
    sp = SamplingParams(max_tokens=6)
    a = Executor(model, max_batch=4, max_ctx=64, use_graphs=False).generate_batch(prompts, sp, prefill_budget=4096)
    b = Executor(model, max_batch=4, max_ctx=64, use_graphs=False).generate_batch(prompts, sp, prefill_budget=8)
    assert [r.output_ids for r in a] == [r.output_ids for r in b]
    assert all(len(r.output_ids) == 6 and r.finish_reason == "length" for r in a)


def test_nvfp4_model_runs_cpu():
    t = dense_tiny()
    model = DenseModel(t, "cpu", seed=1)
    ex = Executor(model, max_batch=2, max_ctx=64, use_graphs=False)
    out = ex.generate_batch(_prompts(2, 9, t.vocab), SamplingParams(max_tokens=3))
    assert all(len(r.output_ids) == 3 for r in out)
    ex.state.check()
    ex.state.cache.flush()
    assert ex.kv.free_count == ex.kv.slots


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["bf16", "nvfp4"])
def test_gpu_matches_cpu_tokens(fmt):
    t = scaled(dense_tiny(), weight_format=fmt)
    cpu = DenseModel(t, "cpu", seed=0)
    gpu = DenseModel(t, "cuda", seed=0, init_device="cpu")
    prompts = _prompts(4, 33, t.vocab)
    sp = SamplingParams(max_tokens=8)
    a = Executor(cpu, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(gpu, max_batch=4, max_ctx=128, use_graphs=True)
    ex.capture_graphs()
    b = ex.generate_batch(prompts, sp)
    agree = sum(x == y for ra, rb in zip(a, b) for x, y in zip(ra.output_ids, rb.output_ids))
    # random-init logits are nearly flat, so a bf16-level difference may flip an argmax now and then;
    # the first token of each request sees identical inputs and must match
    first = sum(ra.output_ids[0] == rb.output_ids[0] for ra, rb in zip(a, b))
    assert first >= (4 if fmt == "bf16" else 3), (first, agree, [r.output_ids for r in a], [r.output_ids for r in b])
    # after the first flip a sequence diverges for good, and FP4 activation rounding amplifies bf16-level noise
    assert agree >= (0.6 if fmt == "bf16" else 0.4) * 32, (first, agree)


@pytest.mark.gpu
def test_graph_equals_eager_gpu():
    t = dense_tiny()
    model = DenseModel(t, "cuda", seed=0, init_device="cpu")
    prompts = _prompts(3, 40, t.vocab)
    sp = SamplingParams(max_tokens=10)
    e1 = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    a = e1.generate_batch(prompts, sp)
    e2 = Executor(model, max_batch=4, max_ctx=128, use_graphs=True)
    e2.capture_graphs()
    b = e2.generate_batch(prompts, sp)
    assert [r.output_ids for r in a] == [r.output_ids for r in b]


def test_dense_model_runs_on_an_nvfp4_kv_cache_cpu():
    """End to end with kv_dtype = nvfp4: the pool holds 4.5 bits per element and generation stays close to the
    bf16-KV run (first tokens equal on this tiny model)."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, t.vocab, (24,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=4)
    bf = Executor(model, max_batch=4, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=64, use_graphs=False, kv_dtype="nvfp4")
    assert ex.kv.fp4
    f4 = ex.generate_batch(prompts, sp)
    assert ex.kv.bytes_per_token == len(t.layers) * 2 * t.kv_heads * (t.head_dim // 2 + t.head_dim // 16)
    assert sum(a.output_ids[0] == b.output_ids[0] for a, b in zip(bf, f4)) >= 2


@pytest.mark.gpu
def test_stable_numerics_makes_verify_rows_bitwise_equal_to_decode_steps():
    """With `stable_numerics` a token's logits do not depend on how many rows share its forward: a 4-row verify
    forward gives, row by row, exactly the bits of four single-token decode steps (split-K and KV-split choices are
    then functions of the layer shape alone)."""
    import torch
    from hibana_b200 import config as cfgmod
    from hibana_b200.engine.context import VERIFY
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import Request, SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny
    t = dense_tiny()
    model = DenseModel(t, "cuda:0", seed=0)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, t.vocab, (300,), generator=g).tolist()
    new = torch.randint(0, t.vocab, (4,), generator=g).tolist()

    def rows_of(stable):
        with cfgmod.using(stable_numerics=stable):
            out = {}
            for mode in ("steps", "verify"):
                ex = Executor(model, max_batch=2, max_ctx=512, use_graphs=False)
                r = Request(prompt_ids=list(prompt), params=SamplingParams(max_tokens=8, ignore_eos=True))
                ex.admit(r)
                ex.prefill_batch([(r, len(prompt))])
                n = len(prompt)
                ex.state.reserve([r], 5)
                ex.runner.set_table(r.table_row, n, r.kv_slots[n:n + 5])
                if mode == "verify":
                    lg, _ = ex.runner.forward_rows([r.table_row], [new], [n], [r.kv_slots[n:n + 4]], mode=VERIFY,
                                                   want="logits_device")
                    out[mode] = lg.float().clone()
                else:
                    rows = []
                    for j, tok in enumerate(new):
                        lg, _ = ex.runner.forward_rows([r.table_row], [[tok]], [n + j], [r.kv_slots[n + j:n + j + 1]],
                                                       mode=VERIFY, want="logits_device")
                        rows.append(lg.float().clone())
                    out[mode] = torch.cat(rows, 0)
            return out
    stable = rows_of(True)
    assert torch.equal(stable["steps"], stable["verify"])
    loose = rows_of(False)          # the default plans may differ by rounding; both must stay close to each other
    assert (loose["steps"] - loose["verify"]).abs().max() <= 0.05 * loose["steps"].abs().max()


def test_w3_decode_copies_serve_decode_and_leave_prefill_alone_cpu():
    """Settings `w3`: every projection gets a 3-bit copy that decode-sized calls use; the prefill chunk above the
    row limit keeps the layer's own weights; generation stays close to the unquantised engine (same first token on
    a bf16 tiny model) and is deterministic."""
    import torch
    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.llm import LLM
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models import linear
    from hibana_b200.target import dense_tiny, scaled
    t = scaled(dense_tiny(), weight_format="bf16")
    # (no prefix cache: a cached prefix shortens the second prefill below the row limit, which then runs on the
    # 3-bit copies: which weights serve a row depends on the call's size, by design of the decode-copy mode)
    cfg = EngineConfig(target="dense-tiny", max_batch=2, cuda_graphs=False, max_context=512, prefill_chunk=512,
                       radix_cache=False)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, t.vocab, (300,), generator=g).tolist()
    plain = LLM(cfg, target=t, device="cpu")
    w3 = LLM(cfg.replace(w3=True), target=t, device="cpu")
    lins = w3.model.linears()
    assert all(l.w3 is not None for l in lins) and all(l.w3 is None for l in plain.model.linears())
    assert lins[0].takes_w3(1) and lins[0].takes_w3(256) and not lins[0].takes_w3(300)
    x = torch.randn(3, t.hidden, generator=g).bfloat16()
    big = torch.randn(linear.W3_MAX_ROWS + 4, t.hidden, generator=g).bfloat16()
    own = plain.model.linears()[0]
    assert torch.equal(lins[0](big), own(big))                       # prefill-sized: the layer's own weights
    err = (lins[0](x).float() - own(x).float()).abs().max() / own(x).float().abs().max()
    assert 0 < err < 0.2                                             # decode-sized: the 3-bit copy (lossy)
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = w3.generate([prompt], sp)[0].output_ids
    b = w3.generate([prompt], sp)[0].output_ids
    assert a == b and len(a) == 6
