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
