import pytest
import torch

from hibana_b200.models.hyper import HyperConnection


def _site(dev, hc=4, h=256, rank=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.1)  # noqa: E731
    return HyperConnection(r(hc * h).to(dev), r(rank, hc * h).to(dev), r(hc * h, rank).to(dev), r(hc, hc * h).to(dev),
                           hc, h), g


def test_mix_combine_semantics_cpu():
    site, g = _site("cpu")
    t, hc, h = 5, 4, 256
    hyper = torch.randn(t, hc * h, generator=g).bfloat16()
    mixed, res = site.mix(hyper)
    assert mixed.shape == (t, h)
    # identical streams and a zero gate projection: the mix is sigmoid(0) * normed = half the normed stream
    site.up.zero_()
    same = torch.randn(t, 1, h, generator=g).expand(t, hc, h).reshape(t, hc * h).bfloat16()
    site.norm.zero_()
    m2, _ = site.mix(same)
    x = same.float().view(t, hc, h)[:, 0]
    want = 0.5 * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + site.eps)
    assert torch.allclose(m2.float(), want, atol=2e-2, rtol=2e-2)
    out = site.combine(torch.ones(t, h).bfloat16(), res)
    assert out.shape == hyper.shape
    delta = (out.float() - hyper.float()).view(t, hc, h)
    assert float(delta.min()) > 0 and float(delta.max()) < 2.0 + 1e-2         # 2 * sigmoid in (0, 2)
    assert float(delta.std(dim=-1).max()) < 2e-2                               # one scalar per (token, stream)


@pytest.mark.gpu
def test_kernels_match_cpu():
    cpu, g = _site("cpu", h=2560, rank=320, seed=3)
    gpu, _ = _site("cuda", h=2560, rank=320, seed=3)
    hyper = torch.randn(37, 4 * 2560, generator=g).bfloat16()
    block = torch.randn(37, 2560, generator=g).bfloat16()
    m_ref, r_ref = cpu.mix(hyper)
    m, r = gpu.mix(hyper.cuda())
    assert torch.allclose(r[1].float().cpu(), r_ref[1].float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(m.float().cpu(), m_ref.float(), atol=3e-2, rtol=3e-2)
    o_ref = cpu.combine(block, r_ref)
    o = gpu.combine(block.cuda(), r)
    assert torch.allclose(o.float().cpu(), o_ref.float(), atol=5e-2, rtol=3e-2)
