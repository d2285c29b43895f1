"""SSD tier: object store (atomic writes, CRCs, epochs, budget), block backup / restore through the KV pool, and the
executor flow (release backs up, a later admission restores instead of re-prefilling)."""
import os

import pytest
import torch

from hibana_b200.cache.kv_pool import KvPool
from hibana_b200.cache.ssd import SsdTier
from hibana_b200.cache.ssd_store import BLOCK_TOKENS, KIND_KV, SsdStore, chain_hash


def test_store_roundtrip_corruption_and_flush(tmp_path):
    st = SsdStore(tmp_path, {"model": "x", "tp_rank": 0})
    key = chain_hash(st.root, list(range(BLOCK_TOKENS)))
    st.write_async(key, KIND_KV, BLOCK_TOKENS, b"a" * 5000, b"meta", token=7)
    st.drain()
    assert st.completions() == [(key, True, 7)]
    hdr, s0, s1 = st.read(key, KIND_KV)
    assert (hdr.tokens, s0, s1) == (BLOCK_TOKENS, b"a" * 5000, b"meta")
    # another identity (e.g. another TP rank) never matches
    other = SsdStore(tmp_path, {"model": "x", "tp_rank": 1})
    assert not other.contains(chain_hash(other.root, list(range(BLOCK_TOKENS))))
    other.close()
    # a restart finds the object again
    st.close()
    st = SsdStore(tmp_path, {"model": "x", "tp_rank": 0})
    assert st.contains(key)
    # damage -> miss, file removed
    path = st._path(key)
    raw = bytearray(path.read_bytes())
    raw[200] ^= 0xFF
    path.write_bytes(bytes(raw))
    assert st.read(key, KIND_KV) is None and not st.contains(key) and st.stats()["corrupt"] == 1
    # flush is an epoch bump: old keys are gone, new root differs
    st.write_async(key, KIND_KV, 1, b"z")
    st.drain()
    root = st.root
    st.flush()
    assert st.root != root and not st.contains(key) and st.stats()["objects"] == 0
    st.close()


def test_store_budget_drops_least_recently_used(tmp_path):
    st = SsdStore(tmp_path, {"m": 1}, budget_bytes=3 * 1200)
    keys = [chain_hash(st.root, [i]) for i in range(5)]
    for k in keys:
        st.write_async(k, KIND_KV, 1, b"x" * 1000)
        st.drain()
    assert not st.contains(keys[0]) and st.contains(keys[-1])
    assert st.stats()["bytes"] <= 3 * 1200
    st.close()


def _tier(tmp_path, slots=2048, **kw):
    kv = KvPool(2, slots, 2, 16, dtype=torch.bfloat16, device="cpu")
    kv.storage.copy_(torch.randn(kv.storage.shape).bfloat16())
    st = SsdStore(tmp_path, {"m": "tiny"}, direct=False)
    return kv, st, SsdTier(st, kv, staging_blocks=4, **kw)


def test_tier_backup_and_restore_blocks(tmp_path):
    kv, st, tier = _tier(tmp_path, min_prefix=512, min_gain=256)
    tokens = list(range(1000, 1000 + 700))
    slots = kv.alloc(700)
    want = kv.rows(slots[:512]).clone()
    assert tier.backup(tokens[:300], slots[:300]) == 0            # below min_prefix
    assert tier.backup(tokens, slots) == 2                         # two whole blocks (+ tail)
    st.drain()
    tier.step()
    assert tier.match(tokens) == 512 and tier.match(tokens[:300]) == 256
    assert tier.worth(tokens, 0) == 512 and tier.worth(tokens, 384) == 0    # gain below min_gain
    tail = tier.read_tail(tokens)
    assert tail is not None and tail[0] == 700 - 512
    # scatter into other slots
    kv.free(slots)
    fresh = kv.alloc(900)[-512:]
    kv.storage.zero_()
    assert tier.restore(tokens, 0, 512, fresh) == 512
    assert torch.equal(kv.rows(fresh), want)
    # a damaged block stops the restore at its start
    key1 = tier._block_keys(tokens, 2)[1]
    p = st._path(key1)
    raw = bytearray(p.read_bytes())
    raw[-10] ^= 1
    p.write_bytes(bytes(raw))
    assert tier.restore(tokens, 0, 512, fresh) == 256
    st.close()


def test_executor_restores_instead_of_reprefilling(tmp_path):
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny
    t = dense_tiny()
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, t.vocab, (600,), generator=g).tolist()
    sp = SamplingParams(max_tokens=4)
    ex = Executor(model, max_batch=2, max_ctx=1024, use_graphs=False)
    ex.enable_ssd_tier(str(tmp_path), min_prefix=256, min_gain=128)
    a = ex.generate_batch([prompt], sp)[0].output_ids
    ex.ssd.store.drain()
    ex.ssd.step()
    assert ex.ssd.stats()["objects"] >= 2
    ex.state.cache.flush()                                   # the GPU cache forgets everything
    before = ex.stats["prefill_tokens"]
    b = ex.generate_batch([prompt], sp)[0].output_ids
    assert ex.stats["ssd_restored_tokens"] == 512
    assert ex.stats["prefill_tokens"] - before == 600 - 512   # only the rest was recomputed
    assert a == b
    ex.ssd.store.close()


@pytest.mark.gpu
def test_kv_copy_kernel_matches_indexing():
    """One launch moves the rows of all layers between the head-major pool and a pinned host payload."""
    kv = KvPool(3, 500, 4, 128, dtype=torch.bfloat16, device="cuda")
    kv.storage.copy_(torch.randn(kv.storage.shape, device="cuda").bfloat16())
    ids = torch.tensor([7, 499, 1, 250, 33], dtype=torch.int32, device="cuda")
    pay = torch.empty(5 * kv.bytes_per_token, dtype=torch.uint8, pin_memory=True)
    kv.copy_payload(ids, pay, to_pool=False)
    torch.cuda.synchronize()
    want = kv.rows(ids.tolist())                                   # [layers, 2, n, heads, d]
    got = pay.view(torch.bfloat16).view(5, 3, 2, 4, 128).permute(1, 2, 0, 3, 4)
    assert torch.equal(got, want.cpu())
    other = torch.tensor([100, 101, 102, 103, 104], dtype=torch.int32, device="cuda")
    kv.copy_payload(other, pay, to_pool=True)
    torch.cuda.synchronize()
    assert torch.equal(kv.rows(other.tolist()), want)


def test_tier_declines_when_recomputing_is_faster(tmp_path):
    """Restore-or-recompute: with measured rates that make a disk read slower than a prefill of the same tokens the
    tier neither restores nor backs up at eviction; unknown rates leave the prefix policy alone."""
    import torch
    from hibana_b200.cache import ssd, ssd_store
    from hibana_b200.cache.kv_pool import KvPool
    kv = KvPool(2, 2048, 2, 64, torch.bfloat16, "cpu")
    store = ssd_store.SsdStore(str(tmp_path), {"t": 1}, budget_bytes=1 << 30)
    tier = ssd.SsdTier(store, kv, min_prefix=256, min_gain=256)
    assert tier.pays(1000)                                   # nothing measured yet
    tier.note_read(10 << 20, 1.0)                            # 10 MB/s disk ...
    tier.note_prefill(4096, 0.05)                            # ... against 82k tokens/s of prefill
    assert not tier.pays(1000)
    toks = list(range(600))
    slots = kv.alloc(600)
    assert tier.backup(toks, slots) > 0                      # explicit backups still work (shutdown persist)
    store.drain()
    tier.step()
    assert tier.match(toks) == 512 and tier.worth(toks, 0) == 0 and tier.declined == 1

    class Node:
        def __init__(self, tokens, slots):
            self.tokens, self.slots, self.parent, self.on_ssd = tokens, slots, type("R", (), {"parent": None})(), False
    other = Node([7] * 600, kv.alloc(600))
    tier.on_evict(other)
    assert not other.on_ssd and tier.declined == 2
    tier.read_gbs, tier.prefill_tok_s = 50.0, 1000.0         # a fast disk against a slow prefill: the tier pays
    assert tier.pays(1000) and tier.worth(toks, 0) == 512
    # before anything was read back, what the writers sustained stands in for the disk's rate: slow writes stop
    # further backups at eviction, and every write is one gathered copy (header, payload, checksum never joined)
    tier.read_gbs, tier.prefill_tok_s = 0.0, 82000.0
    assert store.write_gbs > 0
    store.write_gbs = 0.001
    assert tier.disk_gbs() == pytest.approx(0.001 * len(store._queues)) and not tier.pays(1000)
    third = Node([9] * 600, kv.alloc(600))
    tier.on_evict(third)
    assert not third.on_ssd and tier.declined == 3
    assert store.read(tier._block_keys(toks, 2)[1], ssd_store.KIND_KV) is not None      # round trip of the new writer
