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
