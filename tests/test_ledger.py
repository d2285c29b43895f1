import pytest

from hibana_b200.cache.ledger import GIB, Ledger, graph_bytes


def test_plan_27b_on_180gb():
    # 27B NVFP4: ~16 GiB of weights on a 180 GB part; bf16 KV 64 layers x 8 heads x 128 x 2 x 2 B = 256 KiB / token
    led = Ledger(free_bytes=int(178 * GIB) - 16 * GIB)
    p = led.plan(kv_bytes_per_token=64 * 2 * 8 * 128 * 2, max_batch=64, max_ctx=4096,
                 graph=graph_bytes((1, 2, 4, 8, 16, 32, 64), 5120, 151936, 64))
    assert 400_000 < p.kv_slots < 700_000 and p.state_slots == 0
    assert p.kv_bytes < led.free


def test_state_floor_and_errors():
    led = Ledger(free_bytes=40 * GIB)
    p = led.plan(kv_bytes_per_token=40 * 1024, state_bytes_per_slot=40 << 20, max_batch=64, max_ctx=8192, ssd_restore=True)
    assert p.state_slots == 2 * 64 + 2 and p.kv_slots > 8192
    with pytest.raises(MemoryError):
        Ledger(free_bytes=3 * GIB).plan(kv_bytes_per_token=1024)
    with pytest.raises(MemoryError):
        Ledger(free_bytes=8 * GIB).plan(kv_bytes_per_token=1 << 20, max_ctx=32768)
    small = Ledger(free_bytes=100 * GIB).plan(kv_bytes_per_token=1024, max_batch=2, max_ctx=128)
    assert small.kv_slots == 2 * 128 * 4 and small.notes


def test_speculation_budget_is_set_aside_before_the_pools():
    from hibana_b200.cache.spec_budget import SpecConfig, budget, verify_bytes
    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.llm import plan_memory
    from hibana_b200.target import get_target
    import pytest
    import torch
    t = get_target("nemotron")
    snap = verify_bytes(16, 4, "snapshots", t)
    rec = verify_bytes(16, 4, "reconstruct", t)
    assert snap > 3 * rec > 0                          # replaying compact inputs is what makes deep verify affordable
    fixed, per_slot = budget(SpecConfig("mtp", 3), 16, t)
    assert fixed > rec and per_slot == 2 * t.kv_heads * t.head_dim          # fp8 KV: one byte per element
    assert budget(None, 16, t) == (0, 0)
    with pytest.raises(ValueError):
        SpecConfig("mtp", 9)
    with pytest.raises(ValueError):
        budget(SpecConfig("mtp", 2), 4, get_target("dense-27b"))             # no MTP head
    free = 100 << 30
    cfg = EngineConfig(target="nemotron", max_batch=16, max_context=8192)
    plain = plan_memory(cfg, t, torch.device("cpu"), free_bytes=free)
    spec = plan_memory(cfg.replace(spec="mtp", spec_depth=3), t, torch.device("cpu"), free_bytes=free)
    fixed, _ = budget(SpecConfig("mtp", 3), 16, t, buckets=len(cfg.buckets))
    assert spec["plan"].workspace_bytes - plain["plan"].workspace_bytes == fixed
    assert spec["kv_slots"] <= plain["kv_slots"]
