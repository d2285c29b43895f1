"""MoE routing and grouped expert GEMMs against plain-PyTorch references; EP ranges sum to the whole."""
import pytest
import torch

from hibana_b200.ops import moe


def test_route_ref_properties_cpu():
    lg = torch.randn(7, 16)
    ids, w = moe.route(lg, 4)
    assert ids.shape == (7, 4) and torch.allclose(w.sum(-1), torch.ones(7), atol=1e-5)
    top = torch.topk(torch.softmax(lg, -1), 4).indices
    assert torch.equal(ids.long().sort(-1).values, top.sort(-1).values)
    ids2, w2 = moe.route(lg, 3, sigmoid=True, sel_bias=torch.zeros(16), scale=2.5)
    assert torch.allclose(w2.sum(-1), torch.full((7,), 2.5), atol=1e-4)


def _weights(e, h, inter, act, fmt, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    n1 = 2 * inter if act == "swiglu" else inter
    fc1 = torch.randn(e, n1, h, generator=g) * 0.05
    fc2 = torch.randn(e, h, inter, generator=g) * 0.05
    return moe.ExpertWeights.create(fc1.to(dev), fc2.to(dev), act, fmt, in_amax=5.0, mid_amax=2.0)


def test_experts_ref_ep_halves_sum_cpu():
    ew = _weights(8, 64, 128, "swiglu", "bf16", "cpu")
    x = torch.randn(5, 64).bfloat16()
    ids, w = moe.route(torch.randn(5, 8), 2)
    whole = moe.experts_forward(x, ids, w, ew).float()
    parts = sum(moe.experts_forward(x, ids, w, ew, e_lo=lo, e_n=4).float() for lo in (0, 4))
    assert (whole - parts).abs().max() < 2e-2 * whole.abs().max() + 1e-3
    # a rank that keeps only experts 4..7 (global ids, local weights) computes the same partial sum
    kept = moe.experts_forward(x, ids, w, ew.slice(4, 4), id_base=4).float()
    assert torch.equal(kept, moe.experts_forward(x, ids, w, ew, e_lo=4, e_n=4).float())


@pytest.mark.gpu
@pytest.mark.parametrize("e,k,sig", [(8, 2, False), (512, 10, False), (512, 22, True), (60, 6, True)])
def test_route_gpu(e, k, sig):
    lg = torch.randn(33, e)
    bias = torch.randn(e) * 0.1 if sig else None
    ids, w = moe.route(lg, k, sigmoid=sig, sel_bias=bias, scale=1.7)
    ids_g, w_g = moe.route(lg.cuda(), k, sigmoid=sig, sel_bias=None if bias is None else bias.cuda(), scale=1.7)
    assert torch.equal(ids_g.cpu(), ids)
    assert torch.allclose(w_g.cpu(), w, atol=1e-5, rtol=1e-4)
    if sig:
        # many exactly equal scores around the k-th place: equal scores go to the lower expert index, in both the
        # one-CTA-per-token form (few tokens) and the one-warp-per-token form (many)
        for tokens in (7, 300):
            coarse = (torch.randn(tokens, e) * 2).round() / 2
            ids, w = moe.route(coarse, k, sigmoid=True, scale=1.0)
            ids_g, w_g = moe.route(coarse.cuda(), k, sigmoid=True, scale=1.0)
            assert torch.equal(ids_g.cpu(), ids)
            assert torch.allclose(w_g.cpu(), w, atol=1e-5, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["bf16", "nvfp4", "w3"])
@pytest.mark.parametrize("t,e,k,h,inter,act", [(4, 8, 2, 256, 512, "swiglu"), (37, 16, 4, 256, 128, "relu2"),
                                               (300, 8, 2, 128, 256, "swiglu")])
def test_experts_forward_gpu(fmt, t, e, k, h, inter, act):
    ew = _weights(e, h, inter, act, fmt, "cpu", seed=1)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(t, h, generator=g).bfloat16()
    ids, w = moe.route(torch.randn(t, e, generator=g), k)
    shared = torch.randn(t, h, generator=g).bfloat16()
    ref = moe.experts_forward(x, ids, w, ew, shared=shared).float()
    ewg = ew.to("cuda")
    got = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg, shared=shared.cuda()).float().cpu()
    tol = 3e-2 if fmt == "bf16" else 6e-2
    assert (got - ref).abs().max() <= tol * ref.abs().max() + 2e-3, (got - ref).abs().max()
    # expert-parallel ranges produce partial sums that add up to the whole
    lo = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg, e_lo=0, e_n=e // 2).float()
    hi = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg, e_lo=e // 2, e_n=e // 2).float()
    whole = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg).float()
    assert (lo + hi - whole).abs().max() <= 2e-2 * whole.abs().max() + 2e-3
    if fmt != "w3":    # a rank holding only the upper half of the experts: same partial sum from global ids
        kept = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg.slice(e // 2, e // 2), id_base=e // 2).float()
        assert torch.equal(kept, hi)
    # deterministic
    again = moe.experts_forward(x.cuda(), ids.cuda(), w.cuda(), ewg).float()
    assert torch.equal(again, whole)
    from hibana_b200 import _native as nv
    assert nv.read_status() == 0


def _share_case(seed=0, rows=12, e=64, k=6):
    g = torch.Generator().manual_seed(seed)
    ids, w = moe.route(torch.randn(rows, e, generator=g) * 2, k, sigmoid=True, scale=2.5)
    return ids, w


def test_expert_sharing_keeps_the_budget_and_the_guaranteed_choices_cpu():
    ids, w = _share_case()
    e, k, keep, budget = 64, 6, 2, 30
    assert len(set(ids.flatten().tolist())) > budget
    ids2, w2 = moe.share_experts(ids, w, e, keep, budget, scale=2.5)
    used = {int(ids2[r, j]) for r in range(ids.shape[0]) for j in range(k) if float(w2[r, j]) > 0}
    core = {int(x) for x in ids[:, :keep].flatten()}
    assert core <= used and len(used) <= max(budget, len(core))
    for r in range(ids.shape[0]):
        assert ids2[r, :keep].tolist() == ids[r, :keep].tolist()            # every row keeps its best choices
        live = w2[r] > 0
        assert abs(float(w2[r][live].sum()) - 2.5) < 1e-5                    # renormalised, router scale kept
        kept = [int(x) for x in ids2[r][live]]
        assert kept == [int(x) for x in ids[r] if int(x) in kept]            # rank order preserved
        assert all(int(x) == int(ids[r, 0]) for x in ids2[r][~live])         # lost slots: best expert, weight 0
    # a budget that covers everything changes nothing but the renormalisation
    ids3, w3 = moe.share_experts(ids, w, e, keep, 64, scale=2.5)
    assert torch.equal(ids3, ids) and torch.allclose(w3, w, atol=1e-6)


@pytest.mark.gpu
def test_expert_sharing_kernel_matches_reference():
    for seed, rows, e, k, keep, budget in ((0, 12, 64, 6, 2, 20), (1, 16, 512, 22, 4, 128), (2, 3, 512, 10, 1, 8)):
        ids, w = _share_case(seed, rows, e, k)
        want_i, want_w = moe.share_experts(ids, w, e, keep, budget, scale=1.7)
        got_i, got_w = moe.share_experts(ids.cuda(), w.cuda(), e, keep, budget, scale=1.7)
        assert torch.equal(got_i.cpu(), want_i)
        assert torch.allclose(got_w.cpu(), want_w, atol=1e-6)
