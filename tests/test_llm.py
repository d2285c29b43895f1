"""The engine built from settings: checkpoint loading, the memory plan, the SSD tier as a pipeline."""
import os

import pytest
import torch

from hibana_b200 import config as cfgmod
from hibana_b200.cache.ssd_store import BLOCK_TOKENS
from hibana_b200.engine import llm as llm_mod
from hibana_b200.engine.executor import Executor
from hibana_b200.engine.llm import LLM
from hibana_b200.engine.request import Request, SamplingParams
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, get_target, scaled
from hibana_b200.weights import checkpoint


def test_weights_setting_loads_the_checkpoint_and_reproduces_tokens(tmp_path):
    t = scaled(dense_tiny(), weight_format="nvfp4")
    model = DenseModel(t, "cpu", seed=3)
    checkpoint.save_dense(model, str(tmp_path), hf_layout=True)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, t.vocab, (24,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=6)
    cfg = cfgmod.EngineConfig(max_batch=4, max_context=128, cuda_graphs=False)
    a = [r.output_ids for r in LLM(cfg, target=t, device="cpu", model=model).generate(prompts, sp)]
    b = [r.output_ids for r in LLM(cfg.replace(weights=str(tmp_path)), target=t, device="cpu").generate(prompts, sp)]
    assert a == b
    with pytest.raises(FileNotFoundError):
        LLM(cfg.replace(weights=str(tmp_path / "nothing")), target=t, device="cpu")


def test_memory_plan_sizes_pools_from_free_memory():
    t = get_target("dense-27b")
    cfg = cfgmod.EngineConfig(max_batch=64)
    free = 150 << 30
    mem = llm_mod.plan_memory(cfg, t, torch.device("cpu"), free_bytes=free)
    plan = mem["plan"]
    assert mem["max_ctx"] == t.max_context                       # the native context, not a silent 8192
    per_tok = t.kv_bytes_per_token
    assert mem["kv_slots"] * per_tok < free * cfg.gpu_memory_fraction
    assert mem["kv_slots"] * per_tok > 0.7 * free                # the pool takes what is left, not batch x ctx
    assert plan.kv_slots >= mem["max_ctx"] + 64
    small = llm_mod.plan_memory(cfg, t, torch.device("cpu"), free_bytes=40 << 30)
    assert small["max_ctx"] < t.max_context and any("context limit reduced" in n for n in small["plan"].notes)
    with pytest.raises(MemoryError):                              # an explicit context is a requirement
        llm_mod.plan_memory(cfg.replace(max_context=262144), t, torch.device("cpu"), free_bytes=40 << 30)
    hy = get_target("nemotron")
    m2 = llm_mod.plan_memory(cfgmod.EngineConfig(max_batch=16), hy, torch.device("cpu"), free_bytes=100 << 30)
    assert m2["state_slots"] >= 2 * 16 + 1


def _executor(t, model, tmp, slots=3 * BLOCK_TOKENS + 40, **kw):
    ex = Executor(model, max_batch=2, max_ctx=3 * BLOCK_TOKENS + 64, kv_slots=slots, use_graphs=False)
    ex.enable_ssd_tier(str(tmp), min_prefix=BLOCK_TOKENS, min_gain=BLOCK_TOKENS, **kw)
    return ex


def test_ssd_tier_eviction_backup_async_restore_and_restart(tmp_path):
    """A long prefix is pushed out of the GPU cache by another request: the eviction hook backs it up first, the
    next request with that prefix waits in `can_admit` while the blocks come back asynchronously, its tokens equal
    the uncached run's, the restored rows are byte-equal to the originals, and a new process (a fresh Executor on
    the same directory) finds the prefix after `persist_prefixes` + `rebuild_from_ssd`."""
    t = scaled(dense_tiny(), weight_format="bf16")
    model = DenseModel(t, "cpu", seed=0)
    g = torch.Generator().manual_seed(9)
    long_a = torch.randint(0, t.vocab, (2 * BLOCK_TOKENS + 17,), generator=g).tolist()
    long_b = torch.randint(0, t.vocab, (2 * BLOCK_TOKENS + 5,), generator=g).tolist()
    sp = SamplingParams(max_tokens=4)
    ref = Executor(model, max_batch=2, max_ctx=3 * BLOCK_TOKENS + 64, use_graphs=False).generate_batch([long_a], sp)
    ex = _executor(t, model, tmp_path)
    first = ex.generate_batch([long_a], sp)[0]
    assert first.output_ids == ref[0].output_ids
    rows_before = ex.kv.rows(ex.state.cache.match(long_a[:2 * BLOCK_TOKENS], split=False).slots)
    ex.generate_batch([long_b], sp)                   # does not fit beside A: A's path is evicted -> backed up
    ex.ssd.store.drain()
    ex.ssd.step()
    assert ex.ssd.match(long_a) == 2 * BLOCK_TOKENS
    assert ex.state.cache.match(long_a, split=False).length < BLOCK_TOKENS
    req = Request(prompt_ids=list(long_a), params=sp)
    polls = 0
    while not ex.can_admit(req):                      # the engine would keep stepping other requests meanwhile
        polls += 1
        assert polls < 100000
    got = ex.state.cache.match(long_a[:2 * BLOCK_TOKENS], split=False)
    assert got.length == 2 * BLOCK_TOKENS
    assert torch.equal(ex.kv.rows(got.slots), rows_before)        # restored KV is byte-equal
    cached0 = ex.stats["cached_tokens"]
    again = ex.generate_batch_requests([req])[0]
    assert again.output_ids == ref[0].output_ids and ex.stats["cached_tokens"] - cached0 >= 2 * BLOCK_TOKENS
    assert ex.stats["ssd_restored_tokens"] == 2 * BLOCK_TOKENS
    # shutdown + restart
    assert ex.persist_prefixes() >= 0
    ex.ssd.store.close()
    ex2 = _executor(t, model, tmp_path)
    info = ex2.rebuild_from_ssd()
    assert ex2.stats["ssd_objects_at_start"] >= 2 and info["objects"] >= 2
    ex2.generate_batch([long_b], sp)
    assert ex2.stats["cached_tokens"] >= 2 * BLOCK_TOKENS and ex2.stats["ssd_restored_tokens"] == 2 * BLOCK_TOKENS


def test_llm_enables_the_tier_from_settings(tmp_path):
    t = scaled(dense_tiny(), weight_format="bf16")
    cfg = cfgmod.EngineConfig(max_batch=2, max_context=3 * BLOCK_TOKENS, cuda_graphs=False, ssd_dir=str(tmp_path),
                              ssd_min_prefix=BLOCK_TOKENS, ssd_min_gain=BLOCK_TOKENS, kv_pages=4 * BLOCK_TOKENS)
    llm = LLM(cfg, target=t, device="cpu")
    assert llm.executor.ssd is not None and llm.executor.state.cache.ssd_hook is not None
    g = torch.Generator().manual_seed(2)
    p = torch.randint(0, t.vocab, (BLOCK_TOKENS + 30,), generator=g).tolist()
    llm.generate([p], SamplingParams(max_tokens=2))
    llm.shutdown()
    assert llm.executor.ssd.match(p) == BLOCK_TOKENS
    assert os.listdir(tmp_path)
