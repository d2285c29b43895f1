import pytest
import torch

from hibana_b200.models.qsa import QD, QsaIndexer
from hibana_b200.ops import attention


def _case(dev, lens=(37, 150), ratio=4, budget=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    slots = sum(lens) + 9
    raw = (torch.randn(slots, QD, generator=g)).bfloat16()
    perm = torch.randperm(slots - 1, generator=g) + 1
    table = torch.zeros(len(lens), max(lens), dtype=torch.int32)
    o = 0
    for b, n in enumerate(lens):
        table[b, :n] = perm[o:o + n].int()
        o += n
    ix = QsaIndexer(ratio=ratio, budget=budget, heads=4, rot=64, device=dev)
    ix.norm_w = (torch.randn(QD, generator=g) * 0.1).bfloat16().to(dev)
    first = torch.zeros(len(lens), dtype=torch.int32)
    count = torch.tensor([n // ratio for n in lens], dtype=torch.int32)
    rows_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)])
    rows_pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    q = torch.randn(sum(lens), 4, QD, generator=g).bfloat16()
    return ix, raw, table, first, count, rows_seq, rows_pos, q


def test_selection_rule_cpu():
    ix, raw, table, first, count, rs, rp, q = _case("cpu")
    ckey = torch.zeros_like(raw)
    ix.compress(raw, ckey, table, None, first, count)
    sel, ln = ix.select(q, ckey, table, rs, rp, 149)
    # short context: everything is kept (dense causal): row i of sequence 0 sees exactly tokens 0..i
    for i in (0, 3, 17, 31):
        assert sorted(sel[i, :int(ln[i])].tolist()) == sorted(table[0, :i + 1].tolist())
    # long context: budget // ratio groups + tail
    r = 37 + 149
    assert int(ln[r]) == 32 + (149 + 1 - 150 // 4 * 4)
    tail = table[1, 148:150].tolist()
    assert sel[r, int(ln[r]) - 2:int(ln[r])].tolist() == tail
    # sparse attention over the list equals dense attention restricted to the same tokens
    kp = torch.randn(raw.shape[0], 2, 64).bfloat16()
    vp = torch.randn(raw.shape[0], 2, 64).bfloat16()
    qq = torch.randn(q.shape[0], 4, 64).bfloat16()
    out = QsaIndexer.sparse_attention(qq, kp, vp, sel, ln)
    sl = sel[r, :int(ln[r])].long()
    s = torch.einsum("hd,chd->hc", qq[r].float().view(2, 2, 64).reshape(4, 64),
                     kp[sl].float().repeat_interleave(2, 1)) / 8.0
    want = torch.einsum("hc,chd->hd", torch.softmax(s, -1), vp[sl].float().repeat_interleave(2, 1))
    assert torch.allclose(out[r].float(), want, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_kernels_match_reference():
    ix, raw, table, first, count, rs, rp, q = _case("cpu", lens=(61, 300), budget=64, seed=4)
    ckey = torch.zeros_like(raw)
    ix.compress(raw, ckey, table, None, first, count)
    sel, ln = ix.select(q, ckey, table, rs, rp, 299)
    gx, _, _, _, _, _, _, _ = _case("cuda", lens=(61, 300), budget=64, seed=4)
    ck_g = torch.zeros_like(raw).cuda()
    gx.compress(raw.cuda(), ck_g, table.cuda(), None, first.cuda(), count.cuda())
    used = torch.cat([table[b, :n // 4 * 4:4] for b, n in enumerate((61, 300))]).long()
    assert torch.allclose(ck_g.cpu()[used].float(), ckey[used].float(), atol=2e-2, rtol=2e-2)
    # selection with the SAME compressed keys: the chosen token sets agree (ties aside)
    sel_g, ln_g = gx.select(q.cuda(), ckey.cuda(), table.cuda(), rs.cuda(), rp.cuda(), 299)
    assert torch.equal(ln_g.cpu(), ln)
    agree = 0
    for r in range(q.shape[0]):
        a, b = set(sel[r, :int(ln[r])].tolist()), set(sel_g[r, :int(ln[r])].cpu().tolist())
        agree += len(a & b) / max(len(a), 1)
    assert agree / q.shape[0] > 0.97


def test_indexer_in_the_engine_equals_dense_attention_within_its_budget_cpu():
    """A target with the sparse-attention indexer, served by the engine: while a context has no more groups than the
    budget holds, every token equals the dense engine's (the indexer keeps everything); with a budget far below
    the context the engine still decodes, attending to the selected groups only."""
    import torch
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import ATTN, MLP, Target
    from dataclasses import replace

    def target(**kw):
        return Target(name="qsa-tiny", family="hybrid_moe", hidden=256, vocab=2048, layers=((ATTN, MLP),) * 2,
                      q_heads=4, kv_heads=2, head_dim=64, rope_theta=1e4, ffn=512, max_context=512,
                      prefill_chunk=64, **kw)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (70, 37)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    wide = target(qsa_ratio=4, qsa_budget=128, qsa_heads=2)
    model = HybridModel(wide, "cpu", seed=0)
    ex = Executor(model, max_batch=2, max_ctx=160, use_graphs=False)
    assert ex.runner.qsa and len(ex.kv.idx_raw) == 2
    sparse = [r.output_ids for r in ex.generate_batch(prompts, sp)]
    assert float(ex.kv.idx_key[0].abs().sum()) > 0                 # compressed index keys were written
    dense_ex = Executor(model, max_batch=2, max_ctx=100, use_graphs=False)          # contexts fit the budget: off
    assert not dense_ex.runner.qsa
    dense = [r.output_ids for r in dense_ex.generate_batch(prompts, sp)]
    assert sparse == dense
    # a budget of 16 tokens against 70-token contexts: really sparse now
    model.target = replace(wide, qsa_budget=16)
    for b in model.blocks:
        b.mixer.t = model.target
        b.mixer.indexer.budget = 16
    tight = Executor(model, max_batch=2, max_ctx=160, use_graphs=False)
    out = tight.generate_batch(prompts, sp)
    assert all(len(r.output_ids) == 6 for r in out)
    assert [r.output_ids for r in out] != dense


@pytest.mark.gpu
def test_indexer_in_the_engine_on_gpu_with_graphs():
    """Same rule on the GPU (index-key compression, scoring, top-k, per-row slot lists inside the captured decode
    step): within the budget the tokens are the dense engine's; the status word stays clear."""
    import torch
    from hibana_b200 import _native as nv
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import ATTN, MLP, Target
    t = Target(name="qsa-tiny", family="hybrid_moe", hidden=256, vocab=2048, layers=((ATTN, MLP),) * 2, q_heads=4,
               kv_heads=2, head_dim=128, rope_theta=1e4, ffn=512, max_context=1024, prefill_chunk=128,
               qsa_ratio=4, qsa_budget=256, qsa_heads=2)
    model = HybridModel(t, "cuda:0", seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (150, 61, 200)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    dense_ex = Executor(model, max_batch=4, max_ctx=240, use_graphs=True)
    dense_ex.capture_graphs()
    assert not dense_ex.runner.qsa
    dense = [r.output_ids for r in dense_ex.generate_batch(prompts, sp)]
    ex = Executor(model, max_batch=4, max_ctx=320, use_graphs=True)
    assert ex.runner.qsa
    ex.capture_graphs()
    got = [r.output_ids for r in ex.generate_batch(prompts, sp)]
    torch.cuda.synchronize()
    assert nv.read_status() == 0
    assert got == dense
