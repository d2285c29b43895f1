"""Lock-step control plane for tensor-parallel ranks.

Rank 0 owns HTTP and the inbox; at every publish point of the engine loop it broadcasts the list of commands it is
about to apply over a CPU (gloo) group and every other rank applies the same list, so all schedulers step
identically and sample identical tokens without exchanging them. `serve_rank` is the per-rank entry the
supervisor spawns. Reference: hibana/engine/loop.py:163-182, docs/tensor-parallel.md:53-60.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


class BroadcastChannel:
    """Commands are plain picklable tuples; tickets and notifiers never cross ranks."""

    def __init__(self, group=None, src: int = 0):
        self.group, self.src = group, src

    def broadcast(self, obj=None):
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]


def serve_rank(cfg) -> int:
    """One rank of a tensor-parallel server (rank 0 also serves HTTP)."""
    from ..api.chat_template import ChatTemplate
    from ..api.server import create_app
    from ..engine.executor import Executor
    from ..engine.loop import EngineLoop
    from ..engine.scheduler import Scheduler, SchedulerConfig
    from ..models.dense import DenseModel
    from ..target import get_target
    from ..tokenizer import load_tokenizer
    from .comm import Communicator

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    control = dist.new_group(backend="gloo")
    cfg = BroadcastChannel(control).broadcast(cfg if rank == 0 else None)     # every rank serves rank 0's settings
    comm = Communicator.create(rank, world, dev, slot_mb=cfg.comm_buffer_mb // 8 or 1, timeout_ms=cfg.comm_timeout_ms,
                               fused=cfg.fused_collectives)
    target = get_target(cfg.target)
    if target.family != "dense":
        raise NotImplementedError("tensor-parallel serving covers the dense family; MoE families use expert parallelism")
    model = DenseModel.sharded(target, world, rank, dev, seed=cfg.seed)
    ctx = cfg.max_context or min(target.max_context, 8192)
    ex = Executor(model, max_batch=cfg.max_batch, max_ctx=ctx, kv_slots=cfg.kv_pages, use_graphs=cfg.cuda_graphs,
                  buckets=cfg.buckets, radix_cache=cfg.radix_cache, comm=comm)
    if cfg.cuda_graphs:
        ex.capture_graphs()
    sched = Scheduler(ex, SchedulerConfig(prefill_chunk=cfg.prefill_chunk or target.prefill_chunk,
                                          prefill_budget=cfg.prefill_budget, max_batch=cfg.max_batch,
                                          max_queue=cfg.max_queue))
    engine = EngineLoop(sched, channel=BroadcastChannel(control), rank=rank).start()
    if rank != 0:
        engine.thread.join()
        os._exit(0 if engine.healthy else 1)
    import uvicorn
    tok = load_tokenizer(cfg.weights if cfg.weights != "random" else None, target.vocab)
    app = create_app(engine, tok, model_name=target.name, template=ChatTemplate(),
                     info={"config": cfg.as_dict(), "tp": world}, api_key=cfg.api_key)
    uvicorn.Server(uvicorn.Config(app, host=cfg.host, port=cfg.port, log_level="warning")).run()
    engine.stop()
    os._exit(0)
