"""Expert-parallel all-to-all (parallel/ep.py): fused peer-memory path vs the NCCL counterpart vs a CPU oracle."""
import json
import os
import subprocess
import sys

import pytest
import torch

from hibana_b200.ops import moe

WORKER = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["HB_ROOT"])
from hibana_b200 import _native as nv
from hibana_b200.ops import moe
from hibana_b200.parallel.ep import ExpertParallel
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
res = {}
for fmt, act, E, topk, H, I, toks in (("nvfp4", "swiglu", 16, 4, 256, 128, (37, 50)), ("bf16", "relu2", 8, 2, 128, 128, (5, 0)),
                                      ("nvfp4", "swiglu", 64, 6, 512, 256, (300, 290))):
    g = torch.Generator().manual_seed(3)
    n1 = 2 * I if act == "swiglu" else I
    fc1 = torch.randn(E, n1, H, generator=g) * 0.05
    fc2 = torch.randn(E, H, I, generator=g) * 0.05
    e_per = E // world
    ew = moe.ExpertWeights.create(fc1[rank * e_per:(rank + 1) * e_per].to(dev), fc2[rank * e_per:(rank + 1) * e_per].to(dev), act, fmt)
    full = moe.ExpertWeights.create(fc1.to(dev), fc2.to(dev), act, fmt)
    ep = ExpertParallel.create(rank, world, dev, tokens=max(toks), topk=topk, experts=E, hidden=H, fmt=fmt)
    outs = []
    for call in range(3):                      # consecutive calls reuse the single buffers
        gt = torch.Generator().manual_seed(100 * rank + call)
        t = toks[rank]
        x = (torch.randn(t, H, generator=gt)).bfloat16().to(dev)
        ids, w = moe.route(torch.randn(t, E, generator=gt).to(dev), topk) if t else (torch.empty(0, topk, dtype=torch.int32, device=dev), torch.empty(0, topk, device=dev))
        shared = torch.randn(t, H, generator=gt).bfloat16().to(dev) if call == 1 else None
        a = ep.forward(x, ids, w, ew, shared=shared)
        b = ep.forward_nccl(x, ids, w, ew, shared=shared)
        c = moe.experts_forward(x, ids, w, full, shared=shared) if t else a   # all experts on one GPU
        torch.cuda.synchronize()
        def err(u, v):
            return float((u.float() - v.float()).abs().max() / v.float().abs().max().clamp_min(1e-6)) if u.numel() else 0.0
        outs.append([err(a, b), err(a, c)])
    res[f"{fmt}-{act}-{E}"] = outs
# a whole MoE layer (router, shared expert, routed experts) with this rank's own tokens
from hibana_b200.models.layers import Init, MoeLayer
from hibana_b200.target import flashnext, scaled
t = scaled(flashnext(), hidden=256, experts=16, top_k=4, expert_ffn=128, shared_ffn=128, weight_format="nvfp4")
whole = MoeLayer(t, Init(0, dev, init_device="cpu"), "moe")
layer = MoeLayer(t, Init(0, dev, init_device="cpu"), "moe", ep_rank=rank, ep_size=world)   # keeps its expert range
ep = ExpertParallel.create(rank, world, dev, tokens=64, topk=t.top_k, experts=t.experts, hidden=t.hidden)
xs = torch.randn(40 + 9 * rank, t.hidden, generator=torch.Generator().manual_seed(50 + rank)).bfloat16().to(dev)
a = layer.forward_a2a(xs, ep)
c = whole.forward(xs)
torch.cuda.synchronize()
res["layer"] = [[0.0, float((a.float() - c.float()).abs().max() / c.float().abs().max())]]
res["status"] = nv.read_status(dev)
# a receive buffer that is too small: nothing is written past it, the call ends, and the status word says why
small = ExpertParallel.create(rank, world, dev, tokens=300, topk=4, experts=16, hidden=256, fmt="bf16", rows_cap=256)
g = torch.Generator().manual_seed(9)
fc1 = torch.randn(16, 256, 256, generator=g) * 0.05
fc2 = torch.randn(16, 256, 128, generator=g) * 0.05
ew = moe.ExpertWeights.create(fc1[rank * 8:(rank + 1) * 8].to(dev), fc2[rank * 8:(rank + 1) * 8].to(dev), "swiglu", "bf16")
x = torch.randn(300, 256, generator=g).bfloat16().to(dev)
ids, w = moe.route(torch.randn(300, 16, generator=g).to(dev), 4)
small.forward(x, ids, w, ew)
torch.cuda.synchronize()
res["overflow_status"] = nv.read_status(dev)
gathered = [None] * world
dist.all_gather_object(gathered, res)
if rank == 0:
    print("RESULT " + json.dumps(gathered), flush=True)
dist.barrier()
torch.cuda.synchronize()
os._exit(0)
"""


@pytest.mark.gpu
@pytest.mark.multigpu
def test_ep_all_to_all_matches_nccl_and_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, HB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                          capture_output=True, text=True, env=env, timeout=240)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1]
    ranks = json.loads(line[len("RESULT "):])
    for r in ranks:
        assert r.pop("status") == 0
        assert r.pop("overflow_status") == 10          # kOverflow: raised instead of silently dropping rows
        for name, outs in r.items():
            for e_nccl, e_single in outs:
                assert e_nccl < 3e-2 and e_single < 3e-2, (name, outs)


def test_layout_is_aligned_and_disjoint():
    from hibana_b200 import _native as nv
    if not nv.available():
        pytest.skip("native library not built")
    from hibana_b200.parallel.ep import ExpertParallel
    off, total = ExpertParallel.plan_layout(8, 64, 10, 512, 2560, 2560, "nvfp4", 8192)
    vals = sorted(off.values())
    assert all(v % 1024 == 0 for v in vals) and vals[0] >= 128 and total > vals[-1]
    assert len({v for k, v in off.items() if k != "recv_bf"}) == len(off) - 1   # only the unused buffer aliases
