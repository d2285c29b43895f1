"""Executor: turns scheduler decisions (admit / prefill chunk / decode step / release) into model forwards.

Owns the model, the KV and recurrent-state pools, the StateManager (resource ownership + radix prefix cache) and
the ModelRunner (device block table, graphs). All methods run on the single engine thread.
Reference: hibana/engine/executor.py:51-884 (`admit`, `prefill_batch`, `decode_step`, `release`,
`capture_graphs`, `warmup`, `generate_batch`).
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import torch

from .. import config as cfgmod
from ..cache.kv_pool import KvPool
from ..cache.request_state import StateManager
from ..target import Target
from .context import PREFILL
from ..utils import nvtx
from .request import Request, SamplingParams, State
from .runner import ModelRunner


def _sampling_rows(reqs: Sequence[Request]) -> Optional[dict]:
    if all(r.params.greedy for r in reqs):
        return None
    return {
        "temp": [0.0 if r.params.greedy else r.params.temperature for r in reqs],
        "top_k": [r.params.top_k for r in reqs],
        "top_p": [r.params.top_p for r in reqs],
        "seed": [r.seed & 0x7FFFFFFFFFFFFFFF for r in reqs],
        "offs": [r.draws for r in reqs],
    }


class Executor:
    def __init__(self, model, *, max_batch: int = 64, max_ctx: int = 4096, kv_slots: int = 0,
                 use_graphs: bool = True, buckets: Optional[Sequence[int]] = None, radix_cache: bool = True,
                 state_pool=None, comm=None, kv_dtype: Optional[torch.dtype] = None, attn_splits: int = 0,
                 decode_reserve: int = 64, state_slots: int = 0, state_dtype: torch.dtype = torch.float32,
                 state_window: int = 0,
                 debug_sync: bool = False):
        t: Target = model.target
        self.model, self.target = model, t
        self.device = model.device
        self.max_batch, self.max_ctx = max_batch, max_ctx
        if kv_slots <= 0:
            kv_slots = max_batch * max_ctx
        dtype = kv_dtype or {"fp8": torch.float8_e4m3fn, "nvfp4": "nvfp4"}.get(t.kv_dtype, torch.bfloat16)
        kv_layers = getattr(model, "kv_layers", t.attn_layers) + (1 if getattr(model, "mtp", None) is not None else 0)
        self.kv = KvPool(kv_layers, kv_slots, t.kv_heads, t.head_dim, dtype, self.device) if kv_layers \
            else KvPool(0, kv_slots, 1, 1, dtype, self.device)
        spec = model.state_pool_spec() if hasattr(model, "state_pool_spec") else None
        if state_pool is None and spec is not None:
            from ..cache.state_pool import StatePool
            state_pool = StatePool(spec["layers"], state_slots or (3 * max_batch + 2), spec["conv_dim"],
                                   spec["conv_width"], spec["state_shape"], self.device, state_dtype=state_dtype,
                                   window=state_window if "groups" in spec else 0, groups=spec.get("groups", 1))
        self.state_pool = state_pool
        if state_pool is not None and hasattr(model, "register_state"):
            model.register_state(state_pool)
        buckets = buckets or tuple(b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b <= max_batch)
        self.runner = ModelRunner(model, self.kv, max_batch=max_batch, max_ctx=max_ctx, buckets=buckets,
                                  use_graphs=use_graphs, comm=comm, attn_splits=attn_splits, state_pool=state_pool)
        self.comm = comm
        self.runner.debug_sync = debug_sync
        # sparse-attention indexer: only where a context can outgrow its budget (below that it equals dense attention
        # and would only add kernels); needs x in bf16 at the attention layers, so the trunk keeps the normed rows
        if getattr(t, "qsa_ratio", 0) and max_ctx > t.qsa_budget and kv_layers:
            self.kv.enable_index(kv_layers)
            self.runner.qsa = True
        self.ssd = None
        self._restores: dict = {}        # rid -> RestoreJob in flight, or None once the question is settled
        self.state = StateManager(self.kv, state_pool, cache=radix_cache, decode_reserve=decode_reserve)
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0, "prefill_chunks": 0,
                      "cached_tokens": 0}
        self.spec = None

    def enable_spec(self, depth: int = 2, proposer=None) -> None:
        """Turns on speculative decoding. Drafts come from the model's MTP head, or from `proposer` (a name known
        to proposers.make_proposer, or an object with the engine/contracts.py Proposer interface)."""
        from .spec import SpecDecoder
        if isinstance(proposer, str):
            if proposer == "mtp":
                proposer = None
            else:
                from ..proposers import make_proposer
                proposer = make_proposer(proposer, executor=self)
        self.spec = SpecDecoder(self, depth, proposer=proposer)

    # ---- lifecycle
    def validate_request(self, req: Request) -> None:
        if not req.prompt_ids:
            raise ValueError("empty prompt")
        if req.total_len + req.params.max_tokens > self.max_ctx:
            raise ValueError(f"prompt + max_tokens exceeds the context limit {self.max_ctx}")
        has_media = bool(getattr(req.media, "images", None))
        if any(i >= self.target.vocab or (i < 0 and not has_media) for i in req.prompt_ids):
            raise ValueError("token id out of range")

    def can_admit(self, req: Request, promised: int = 0) -> bool:
        """Pure while no SSD tier is on. With one, the first call for a request may start an asynchronous restore
        of its prefix; the request then stays in the queue (this returns False) while reader threads and scatter
        kernels bring the blocks back, and the engine keeps stepping everybody else."""
        if self.ssd is not None and req.cacheable and not self._restore_settled(req):
            return False
        return bool(self.runner._free_rows) and self.state.can_admit(req, promised)

    def _restore_settled(self, req: Request) -> bool:
        if req.rid in self._restores and self._restores[req.rid] is None:
            return True
        job = self._restores.get(req.rid)
        if job is None:
            self.ssd.step()
            job = self.state.begin_ssd_restore(req.all_ids if req.output_ids else req.prompt_ids, self.ssd)
            self._restores[req.rid] = job
            if job is None:
                return True
        done = self.ssd.pump(job)
        if self.comm is not None:          # ranks finish reads at different times; they move on together
            done = bool(self.comm.min_int(int(done)))
        if not done:
            return False
        got = self.state.finish_ssd_restore(job, self.ssd)
        self.stats["ssd_restored_tokens"] = self.stats.get("ssd_restored_tokens", 0) + got
        self._restores[req.rid] = None
        return True

    def enable_ssd_tier(self, directory: str, *, budget_bytes: int = 200 << 30, min_prefix: Optional[int] = None,
                        min_gain: Optional[int] = None, identity: Optional[dict] = None,
                        trace_path: Optional[str] = None) -> None:
        """Long prefixes are backed up to `directory` when a request is released and when the radix tree evicts
        them, and come back on admission when that gains enough tokens over the GPU cache (cache/ssd.py). With
        tensor parallelism every rank stores its own heads and the ranks agree on how far a restore got."""
        from ..cache import ssd, ssd_store
        t = self.model.target
        ident = {"target": t.name, "layers": len(t.layers), "kv_heads": t.kv_heads, "head_dim": t.head_dim,
                 "kv_dtype": str(self.kv.dtype), "kv_bytes_per_token": self.kv.bytes_per_token,
                 "weight_format": getattr(t, "weight_format", ""),
                 "tp_rank": self.comm.rank if self.comm is not None else 0,
                 "tp_size": self.comm.world if self.comm is not None else 1}
        ident.update(identity or {})
        store = ssd_store.SsdStore(directory, ident, budget_bytes=budget_bytes)
        agree = (lambda n: self.comm.min_int(n)) if self.comm is not None else None
        self.ssd = ssd.SsdTier(store, self.kv, min_prefix=ssd.MIN_PREFIX if min_prefix is None else min_prefix,
                               min_gain=ssd.MIN_GAIN if min_gain is None else min_gain, agree=agree)
        if self.state.cache is not None:
            self.state.cache.ssd_hook = self.ssd.on_evict     # backup before the KV of an evicted path is freed
        if trace_path:
            # one JSON line per restore (how far it got, whether a block was missing): the tier's own event hook
            import json
            import time
            fh = open(trace_path, "a")

            def trace(event: str, **fields):
                fh.write(json.dumps({"t": time.time(), "event": event, **fields}) + "\n")
                fh.flush()
            self.ssd.trace = trace

    def rebuild_from_ssd(self) -> dict:
        """Start-up: indexes what an earlier run left in the tier's directory (objects are content-addressed by the
        chained hash of their tokens, so finding a prefix needs no rebuilt tree, only the key index)."""
        if self.ssd is None:
            return {}
        self.ssd.store.scan()                     # (the store also scans when it is opened)
        self.stats["ssd_objects_at_start"] = self.ssd.store.stats()["objects"]
        return self.ssd.stats()

    def persist_prefixes(self) -> int:
        """Shutdown: every cached path long enough for the tier goes to disk; returns blocks written."""
        if self.ssd is None or self.state.cache is None:
            return 0
        return self.ssd.persist(self.state.cache)

    def warmup(self, prompt_len: int = 64) -> None:
        """One short request through prefill and a few decode steps (all code paths, allocator pools, tensor-map
        cache and graphs touched once) before the first real request pays for it; leaves no trace in the cache."""
        n = max(8, min(prompt_len, self.max_ctx // 4))
        r = Request(prompt_ids=[1 + (i % max(self.target.vocab - 2, 1)) for i in range(n)],
                    params=SamplingParams(max_tokens=4, ignore_eos=True))
        r.cacheable = False
        spec, self.spec = self.spec, None
        try:
            self.generate_batch_requests([r])
        finally:
            self.spec = spec
        for k in self.stats:
            self.stats[k] = 0

    def admit(self, req: Request) -> None:
        """Takes a block-table row (and, with a cache, the matched prefix) for the request."""
        if self.ssd is not None and req.cacheable and req.rid not in self._restores:
            # offline callers admit without asking `can_admit` first: settle the restore question here, blocking
            import time
            while not self._restore_settled(req):
                time.sleep(0.0005)
        self._restores.pop(req.rid, None)
        req.table_row = self.runner.alloc_row()
        try:
            self.state.admit(req)
        except Exception:
            self.runner.free_row(req.table_row)
            req.table_row = -1
            raise
        if req.cached_len:
            self.runner.set_table(req.table_row, 0, req.kv_slots[:req.cached_len])
            self.stats["cached_tokens"] += req.cached_len
        req.prefilled = req.cached_len
        req.state = State.PREFILL
        if req.params.constraint is not None and req.grammar is None:
            from .grammar import GrammarState
            req.grammar = GrammarState(req.params.constraint, self.target.vocab)

    def release(self, req: Request) -> None:
        if req.table_row < 0:
            return
        if getattr(self, "ssd", None) is not None and req.cacheable and req.reserved == 0:
            n = req.committed_len
            self.ssd.backup(req.all_ids[:n], req.kv_slots[:n])
            self.ssd.step()
        self.state.release(req)
        if self.spec is not None:
            self.spec.release(req)
        self.runner.free_row(req.table_row)
        req.table_row = -1

    def retract(self, req: Request) -> None:
        """Drops physical resources; the emitted history stays and is replayed on re-admission."""
        self.state.retract(req)
        if self.spec is not None:
            self.spec.release(req)
        self.runner.free_row(req.table_row)
        req.table_row, req.prefilled, req.committed_len, req.cached_len = -1, 0, 0, 0
        req.state = State.WAITING

    # ---- steps
    def _alloc(self, req: Request, n: int) -> list[int]:
        return self.state.extend(req, n)

    @nvtx.ranged("prefill")
    def prefill_batch(self, chunks: Sequence[tuple[Request, int]]) -> None:
        """Runs `count` more prompt (or replayed) tokens of each request; samples when a prompt completes."""
        t_start = time.perf_counter() if self.ssd is not None else 0.0
        rows, toks, starts, slot_lists, finals = [], [], [], [], []
        taken: list[tuple[Request, int]] = []
        for req, count in chunks:
            seq = req.all_ids if req.output_ids else req.prompt_ids
            # After a retraction the emitted history is replayed; the last emitted token stays pending.
            target_len = len(seq) - (1 if req.output_ids else 0)
            count = min(count, target_len - req.prefilled)
            if self.state_pool is not None and req.prefilled < req.branch_at < req.prefilled + count:
                # stop at the point where this prompt left a cached path, so a state snapshot lands there and the
                # next request sharing that prefix can resume from it
                count = req.branch_at - req.prefilled
            tokens = seq[req.prefilled:req.prefilled + count]
            try:
                slots = self._alloc(req, count)
            except MemoryError:
                for r, n in taken:      # all or nothing: a half-allocated step is never run
                    drop = r.kv_slots[len(r.kv_slots) - n:]
                    del r.kv_slots[len(r.kv_slots) - n:]
                    self.kv.free(drop)
                raise
            taken.append((req, count))
            rows.append(req.table_row)
            toks.append(tokens)
            starts.append(req.prefilled)
            slot_lists.append(slots)
            finals.append(req.prefilled + count >= target_len)
        any_final = any(finals)
        extras = {"want_hidden": True} if self.spec is not None else None
        if any(getattr(r.media, "images", None) for r, _ in chunks):
            # image placeholders inside this step's chunks take the vision encoder's rows (encoded once per image)
            from .media import VisionCache, chunk_embeddings
            if getattr(self, "_vision_cache", None) is None:
                if getattr(self.model, "vision", None) is None:
                    raise ValueError("this target has no vision encoder")
                self._vision_cache = VisionCache(self.model.vision)
            rows_img = [chunk_embeddings(r.media, starts[i], len(toks[i]), self._vision_cache)
                        for i, (r, _) in enumerate(chunks) if getattr(r.media, "images", None)]
            rows_img = [x for x in rows_img if x is not None]
            if rows_img:
                extras = dict(extras or {})
                extras["image_embeds"] = torch.cat(rows_img, 0)
        masks = None
        if any_final and any(r.grammar is not None for r, _ in chunks):
            from .grammar import stack_masks
            masks = stack_masks([r.grammar.mask() if r.grammar is not None and not r.output_ids else None
                                 for r, _ in chunks], (self.target.vocab + 31) // 32)
        lps = [r.params.logprobs if f and not r.output_ids else 0 for (r, _), f in zip(chunks, finals)]
        out = self.runner.forward_rows(rows, toks, starts, slot_lists, mode=PREFILL,
                                       want="last" if any_final else "none", extras=extras, masks=masks,
                                       logprobs=lps if any(lps) else None,
                                       sampling_rows=_sampling_rows([r for r, _ in chunks]) if any_final else None,
                                       state_slots=[r.state_slot for r, _ in chunks]
                                       if self.state_pool is not None else None)
        if self.ssd is not None and any_final:       # a synchronised step: feeds the tier's restore-or-recompute model
            self.ssd.note_prefill(sum(len(x) for x in toks), time.perf_counter() - t_start)
        if self.spec is not None:
            off = 0
            for i, (req, _) in enumerate(chunks):
                n = len(toks[i])
                self.spec.ingest_prefill(req, extras["hidden"][off:off + n], starts[i], n)
                off += n
        for i, (req, _) in enumerate(chunks):
            n = len(toks[i])
            req.prefilled += n
            req.committed_len = req.prefilled
            self.stats["prefill_tokens"] += n
            self.state.after_prefill(req, final=finals[i])
            if finals[i]:
                req.state = State.RUNNING
                if not req.output_ids:      # a replayed request already holds its pending token
                    req.draws += 1
                    if self.runner.last_logprobs and i in self.runner.last_logprobs:
                        req.token_logprobs.append(self.runner.last_logprobs[i])
                    req.push(out[i])
        self.stats["prefill_chunks"] += 1

    @nvtx.ranged("decode")
    def decode_step(self, reqs: Sequence[Request]) -> None:
        """One token for every running request (the pending token goes in, the next one comes out)."""
        if self.spec is not None:     # greedy, relaxed and sampled requests all verify drafts (engine/spec.py)
            self.spec.round(reqs)
            self.stats["decode_steps"] += 1
            self.stats["decode_tokens"] += sum(r.rounds[-1] for r in reqs)
            return
        slots = [s[0] for s in self.state.reserve(reqs, 1)]   # all or nothing; MemoryError -> scheduler retracts
        rows = [r.table_row for r in reqs]
        tokens = [r.output_ids[-1] for r in reqs]
        positions = [r.total_len - 1 for r in reqs]
        masks = [r.grammar.mask() if r.grammar is not None else None for r in reqs]
        lps = [r.params.logprobs for r in reqs]
        out = self.runner.decode(rows, tokens, positions, slots, _sampling_rows(reqs),
                                 [r.state_slot for r in reqs] if self.state_pool is not None else None,
                                 masks if any(m is not None for m in masks) else None,
                                 logprobs=lps if any(lps) else None)
        got = self.runner.last_logprobs or {}
        for i, (r, tok) in enumerate(zip(reqs, out)):
            self.state.commit(r, 1)
            r.draws += 1
            if i in got:
                r.token_logprobs.append(got[i])
            r.push(tok)
        self.stats["decode_steps"] += 1
        self.stats["decode_tokens"] += len(reqs)

    def idle_round(self, state: int = 0) -> list:
        """Data-parallel engine with nothing to run: one lockstep round (and the empty forward it may ask for)."""
        return self.runner.idle_round(state)

    def capture_graphs(self) -> None:
        self.runner.capture()
        if self.spec is not None and getattr(self.spec, "graphs", None) is not None:
            self.spec.graphs.capture()
        if self.spec is not None and getattr(self.spec, "draft_graphs", None) is not None:
            self.spec.draft_graphs.capture()

    # ---- offline batch API
    def generate_batch(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams],
                       prefill_budget: int = 4096) -> list[Request]:
        """Runs prompts to completion with a simple loop (admit all, chunked prefill, lock-step decode)."""
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        return self.generate_batch_requests([Request(prompt_ids=list(p), params=sp) for p, sp in zip(prompts, plist)],
                                            prefill_budget)

    def generate_batch_requests(self, reqs: list, prefill_budget: int = 4096) -> list[Request]:
        for r in reqs:
            self.validate_request(r)
        pending = list(reqs)
        active: list[Request] = []
        while pending or active:
            while pending and len(active) < self.max_batch and self.can_admit(pending[0]):
                r = pending.pop(0)
                self.admit(r)
                active.append(r)
            pre = [r for r in active if r.state == State.PREFILL]
            if pre:
                budget, chunks = prefill_budget, []
                for r in pre:
                    if budget <= 0:
                        break
                    c = min(len(r.prompt_ids) - r.prefilled, budget)
                    chunks.append((r, c))
                    budget -= c
                self.prefill_batch(chunks)
            else:
                run = [r for r in active if r.state == State.RUNNING]
                if run:
                    self.decode_step(run)
            for r in [r for r in active if r.done]:
                self.release(r)
                active.remove(r)
        return reqs
