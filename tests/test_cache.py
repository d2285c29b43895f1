"""Radix cache, StateManager ownership invariants and prefix-cache hits through the executor (CPU)."""
import random

import pytest
import torch

from hibana_b200.cache.kv_pool import KvPool
from hibana_b200.cache.radix import RadixCache, Snapshot
from hibana_b200.cache.request_state import StateManager
from hibana_b200.cache.state_pool import StatePool
from hibana_b200.engine.executor import Executor
from hibana_b200.engine.request import Request, SamplingParams
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled


def test_radix_insert_match_split_evict():
    freed = []
    c = RadixCache(freed.extend)
    a = list(range(10))
    node, adopted = c.insert(a, list(range(100, 110)))
    assert adopted == 10 and c.size == 10
    m = c.match(a[:6] + [99, 98])
    assert m.length == 6 and m.slots == list(range(100, 106))
    c.check()
    lock = c.lock(m.node)
    assert c.evictable_size == 4
    b = a[:6] + [50, 51]
    node2, adopted2 = c.insert(b, list(range(100, 106)) + [200, 201], start=6)
    assert adopted2 == 8 and c.size == 12
    c.check()
    assert c.evict(100) == 6 and sorted(freed) == [106, 107, 108, 109, 200, 201]
    c.unlock(lock)
    c.check()
    assert c.evict(100) == 6 and c.size == 0
    c.check()


def test_radix_duplicate_insert_keeps_private_copy():
    freed = []
    c = RadixCache(freed.extend)
    c.insert([1, 2, 3, 4], [10, 11, 12, 13])
    node, adopted = c.insert([1, 2, 3, 4, 5], [20, 21, 22, 23, 24], start=0)
    assert adopted == 0 and c.size == 4      # the tree already holds other slots for these tokens
    c.check()


def test_radix_snapshots_and_usable_length():
    states = []
    c = RadixCache(lambda s: None, states.append, needs_state=True)
    n1, _ = c.insert(list(range(8)), list(range(8)))
    c.set_snapshot(n1, Snapshot(slot=3, position=8))
    n2, _ = c.insert(list(range(12)), list(range(12)), start=8)
    m = c.match(list(range(12)))
    assert m.length == 12 and m.state_length == 8
    node, length = c.usable(m)
    assert length == 8 and node is n1
    lk = c.lock(node)
    assert c.evict_snapshots(5) == 0
    c.unlock(lk)
    assert c.evict_snapshots(5) == 1 and states == [3]
    m = c.match(list(range(12)))
    assert c.usable(m)[1] == 0 and c.full_reprefills == 1
    c.check()


def _req(tokens, n=4):
    return Request(prompt_ids=list(tokens), params=SamplingParams(max_tokens=n))


def test_state_manager_fuzz_conservation():
    rng = random.Random(7)
    kv = KvPool(1, 400, 1, 4)
    sp = StatePool(1, 12, 4, 4, (2, 2))
    sm = StateManager(kv, sp, cache=True, decode_reserve=4)
    bases = [[rng.randrange(50) for _ in range(30)] for _ in range(3)]
    live = []
    for step in range(400):
        op = rng.random()
        if op < 0.35 and len(live) < 5:
            base = rng.choice(bases)
            toks = base[:rng.randrange(5, 30)] + [rng.randrange(50) for _ in range(rng.randrange(0, 6))]
            r = _req(toks, n=rng.randrange(1, 8))
            if sm.can_admit(r):
                sm.admit(r)
                r.prefilled = r.cached_len
                live.append(r)
        elif op < 0.75 and live:
            r = rng.choice(live)
            if r.prefilled < len(r.prompt_ids):
                n = min(rng.randrange(1, 9), len(r.prompt_ids) - r.prefilled)
                try:
                    sm.extend(r, n)
                except MemoryError:
                    sm.retract(r)
                    live.remove(r)
                    continue
                r.prefilled += n
                r.committed_len = r.prefilled
                final = r.prefilled == len(r.prompt_ids)
                sm.after_prefill(r, final=final)
                if final:
                    r.output_ids.append(rng.randrange(50))
            elif r.remaining > 0:
                try:
                    sm.reserve([r], 3)
                except MemoryError:
                    continue
                keep = rng.randrange(1, 4)
                sm.commit(r, keep)
                for _ in range(keep):
                    r.output_ids.append(rng.randrange(50))
        elif live:
            r = rng.choice(live)
            (sm.release if rng.random() < 0.8 else sm.retract)(r)
            live.remove(r)
        sm.check()
    for r in live:
        sm.release(r)
    sm.check()
    sm.cache.flush()
    assert kv.free_count == kv.slots and sp.free_count == sp.slots


def test_prefix_cache_hit_gives_same_tokens_cpu():
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, t.vocab, (48,), generator=g).tolist()
    prompts = [shared + torch.randint(0, t.vocab, (16,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=5)
    cold = Executor(model, max_batch=4, max_ctx=128, use_graphs=False, radix_cache=False)
    ref = [cold.generate_batch([p], sp)[0].output_ids for p in prompts]
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False, radix_cache=True)
    outs, cached = [], []
    for p in prompts:
        r = ex.generate_batch([p], sp)[0]
        outs.append(r.output_ids)
        ex.state.check()
    assert outs == ref
    assert ex.stats["cached_tokens"] == 48 * 2
    assert ex.state.cache.size > 0
    # a repeated prompt reuses everything but its last token
    before = ex.stats["cached_tokens"]
    again = ex.generate_batch([prompts[0]], sp)[0]
    assert again.output_ids == ref[0] and ex.stats["cached_tokens"] - before == 63
    ex.state.check()


def test_cache_trace_pins_cache_paths_to_the_cold_run(tmp_path):
    """The cache trace: a prefix served from the radix cache, and one restored from the SSD tier, give the same
    first token and bit-equal last-token activations as the cold prefill of an attention-only model."""
    import torch
    from hibana_b200.engine import cache_trace
    from hibana_b200.engine.executor import Executor
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import ATTN, MLP, get_target, scaled
    t = scaled(get_target("tiny"), layers=None, mtp_layers=0, weight_format="bf16")
    t = scaled(t, layers=2)
    import dataclasses
    t = dataclasses.replace(t, layers=((ATTN, MLP), (ATTN, MLP)), ffn=256)
    model = HybridModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(3, t.vocab, (600,), generator=g).tolist()
    make = lambda: Executor(model, max_batch=2, max_ctx=1024, kv_slots=2048, use_graphs=False)  # noqa: E731
    rep = cache_trace.run(make, ids, 520, tmp_path / "trace.json", chunk=64, ssd_dir=str(tmp_path / "ssd"))
    assert rep["cached_prefix"] >= 512 and rep["restored_tokens"] >= 512
    toks = rep["first_tokens"]
    assert toks["cold"] == toks["cached"] == toks["restored"] == toks["chunked"]
    assert rep["pairs"]["cached_vs_cold"]["max_rel_diff"] < 2e-2
    assert rep["pairs"]["restored_vs_cached"]["equal"]            # restore is a byte copy of what the cache held
    assert (tmp_path / "trace.json").exists() and (tmp_path / "trace.pt").exists()
