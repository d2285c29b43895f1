"""Control plane of multi-rank serving: lock-step tensor-parallel ranks, or data-parallel replicas.

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
        """`src`: the sender's rank within `group` (a tensor-parallel group's leader is its rank 0)."""
        self.group, self.src = group, src

    def broadcast(self, obj=None):
        box = [obj]
        dist.broadcast_object_list(box, group_src=self.src, group=self.group)
        return box[0]


class ThreadBroadcast:
    """The same channel between threads of one process (tests): `view(0)` sends, the other views receive."""

    def __init__(self, world: int, timeout: float = 60.0):
        import queue
        self.timeout = timeout
        self.queues = [queue.Queue() for _ in range(world)]

    def view(self, rank: int):
        outer = self

        class _View:
            def broadcast(self, obj=None):
                if rank == 0:
                    for q in outer.queues[1:]:
                        q.put(obj)
                    return obj
                return outer.queues[rank].get(timeout=outer.timeout)
        return _View()


def replica_groups(dp: int, tp: int, rank: int, device_backend: str = "nccl", timeout_s: float = 30.0):
    """Process groups of data-parallel replicas that are tensor-parallel groups: ranks [g * tp, (g + 1) * tp) are
    replica g. Returns (this rank's group for tensor collectives, the same ranks as a host group with a timeout for
    the leader's command broadcast, the host group of the replicas' leaders). Collective over the world: every
    rank creates every group, in the same order."""
    import datetime
    limit = datetime.timedelta(seconds=timeout_s)
    members = [list(range(g * tp, (g + 1) * tp)) for g in range(dp)]
    device = [dist.new_group(ranks=m, backend=device_backend) for m in members]
    host = [dist.new_group(ranks=m, backend="gloo", timeout=limit) for m in members]
    leaders = dist.new_group(ranks=[m[0] for m in members], backend="gloo", timeout=limit)
    return device[rank // tp], host[rank // tp], leaders


def serve_rank(cfg) -> int:
    """One rank of a multi-GPU server (rank 0 also serves HTTP). Tensor parallel (the default), every family: the
    dense decoder and the hybrids shard their mixers by head, MLPs by column and experts by expert range over the
    ranks (`build_model`). With `dp` > 1 the ranks are data-parallel replicas instead, each one GPU or (with `tp` > 1
    too) a tensor-parallel group of `tp` GPUs. The engine stack itself comes from the settings (`LLM`), the same as
    on one GPU."""
    import datetime

    from ..api.chat_template import ChatTemplate
    from ..api.server import create_app
    from ..engine.llm import LLM
    from ..engine.loop import EngineLoop
    from ..tokenizer import load_tokenizer
    from .comm import Communicator
    from .watchdog import PeerWatchdog

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    # the control plane has a timeout: a rank that stops answering ends the others' next broadcast with an error
    control = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=max(cfg.control_timeout_s, 5)))
    cfg = BroadcastChannel(control).broadcast(cfg if rank == 0 else None)     # every rank serves rank 0's settings
    if cfg.dp * cfg.tp != world and cfg.dp > 1:
        raise ValueError(f"dp={cfg.dp} x tp={cfg.tp} does not match the {world} ranks that were started")
    if cfg.dp > 1 and cfg.tp > 1:
        # data-parallel replicas of tensor-parallel groups: ranks [g * tp, (g + 1) * tp) are replica g. The group
        # has its own NCCL group and peer heap; its rank 0 is the replica's leader: it takes part in the replicas'
        # rounds and passes every command it applies on to its followers (engine/loop.py). Every rank takes part in
        # the creation of every group.
        tp, group, tp_rank = cfg.tp, rank // cfg.tp, rank % cfg.tp
        device_group, host_group, leaders = replica_groups(cfg.dp, tp, rank, "nccl", max(cfg.control_timeout_s, 5))
        comm = Communicator.create(tp_rank, tp, dev, slot_mb=cfg.comm_buffer_mb // 8 or 1,
                                   timeout_ms=cfg.comm_timeout_ms, fused=cfg.fused_collectives, group=device_group)
        from ..engine.dp import GroupAllGather
        channel = BroadcastChannel(host_group)
        if tp_rank == 0:
            llm = LLM(cfg, device=dev, comm=comm, control=GroupAllGather(leaders), rank=group, warmup=True)
            engine = EngineLoop(llm.scheduler, channel=channel, rank=group, dp=llm.lockstep).start()
        else:
            llm = LLM(cfg, device=dev, comm=comm, warmup=True)
            engine = EngineLoop(llm.scheduler, channel=channel, rank=tp_rank).start()
    elif cfg.dp > 1:
        # data-parallel replicas (one per GPU), expert-parallel MoE layers between them when cfg.ep == cfg.dp: every
        # replica schedules its own requests; rank 0 routes them and collects the tokens (engine/loop.py, engine/dp.py)
        from ..engine.dp import GroupAllGather
        llm = LLM(cfg, device=dev, control=GroupAllGather(control), rank=rank, warmup=True)
        engine = EngineLoop(llm.scheduler, rank=rank, dp=llm.lockstep).start()
    else:
        comm = Communicator.create(rank, world, dev, slot_mb=cfg.comm_buffer_mb // 8 or 1,
                                   timeout_ms=cfg.comm_timeout_ms, fused=cfg.fused_collectives)
        llm = LLM(cfg.replace(tp=world), device=dev, comm=comm, warmup=True)
        engine = EngineLoop(llm.scheduler, channel=BroadcastChannel(control), rank=rank).start()

    def on_dead(ranks):
        engine._fail(f"ranks {list(ranks)} stopped answering")
        os._exit(13)                      # non-zero: the supervisor restarts the whole group
    store = dist.TCPStore("127.0.0.1", int(os.environ.get("MASTER_PORT", "29500")) + 23, world, rank == 0,
                          timeout=datetime.timedelta(seconds=60))
    PeerWatchdog(store, rank, world, interval=1.0, timeout=float(max(cfg.control_timeout_s, 5)),
                 on_dead=on_dead).start()
    if rank != 0:
        engine.thread.join()
        os._exit(0 if engine.healthy else 1)
    import uvicorn
    tok = load_tokenizer(cfg.weights if cfg.weights != "random" else None, llm.target.vocab)
    app = create_app(engine, tok, model_name=llm.target.name, template=ChatTemplate(),
                     info={"config": cfg.as_dict(), "tp": cfg.tp if cfg.dp > 1 else world, "dp": cfg.dp},
                     api_key=cfg.api_key)
    uvicorn.Server(uvicorn.Config(app, host=cfg.host, port=cfg.port, log_level="warning")).run()
    engine.stop()
    llm.shutdown()
    os._exit(0)
