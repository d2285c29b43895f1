"""Lock-step command broadcast between two CPU ranks (gloo): both schedulers see the same commands."""
import json
import os
import subprocess
import sys

WORKER = r"""
import json, os, queue, sys, time
sys.path.insert(0, os.environ["HB_ROOT"])
sys.path.insert(0, os.path.join(os.environ["HB_ROOT"], "tests"))
import torch.distributed as dist
from hibana_b200.engine.loop import EngineLoop
from hibana_b200.engine.request import SamplingParams
from hibana_b200.engine.scheduler import Scheduler, SchedulerConfig
from hibana_b200.parallel.lockstep import BroadcastChannel
from test_scheduler import FakeExecutor
rank = int(os.environ["RANK"])
dist.init_process_group("gloo")
ex = FakeExecutor()
loop = EngineLoop(Scheduler(ex, SchedulerConfig(max_batch=4)), channel=BroadcastChannel(), rank=rank).start()
outs = []
if rank == 0:
    tickets = [loop.submit([i, i + 1, i + 2], SamplingParams(max_tokens=4)) for i in range(3)]
    for t in tickets:
        toks = []
        while True:
            kind, val = t.events.get(timeout=30)
            if kind == "tokens":
                toks.extend(val)
            else:
                break
        outs.append(toks)
    time.sleep(0.3)
    loop.stop()
else:
    loop.thread.join(30)
decodes = [e for e in ex.log if e[0] == "decode"]
with open(os.environ["HB_OUT"] + f".{rank}", "w") as f:
    json.dump({"outs": outs, "steps": len(ex.log), "decode_batches": [len(d[1]) for d in decodes]}, f)
os._exit(0)
"""


def test_two_cpu_ranks_apply_the_same_commands(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HB_ROOT=root, HB_OUT=str(tmp_path / "out"))
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                       capture_output=True, text=True, env=env, timeout=180)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    r0 = json.loads((tmp_path / "out.0").read_text())
    r1 = json.loads((tmp_path / "out.1").read_text())
    assert len(r0["outs"]) == 3 and all(len(o) == 4 for o in r0["outs"])
    assert r0["steps"] == r1["steps"] and r0["decode_batches"] == r1["decode_batches"]


GROUPS_WORKER = r"""
import json, os, sys, time
sys.path.insert(0, os.environ["HB_ROOT"])
import torch.distributed as dist
from hibana_b200.config import EngineConfig
from hibana_b200.engine.dp import GroupAllGather
from hibana_b200.engine.llm import LLM
from hibana_b200.engine.loop import EngineLoop
from hibana_b200.engine.request import SamplingParams
from hibana_b200.parallel.comm import GlooCommunicator
from hibana_b200.parallel.lockstep import BroadcastChannel, replica_groups
from hibana_b200.target import dense_tiny, scaled
rank = int(os.environ["RANK"])
dist.init_process_group("gloo")
dp, tp = 2, 2
device_group, host_group, leaders = replica_groups(dp, tp, rank, "gloo", 60)
g, r = rank // tp, rank % tp
t = scaled(dense_tiny(), weight_format="bf16")
cfg = EngineConfig(target="dense-tiny", max_batch=4, cuda_graphs=False, max_context=128, prefill_budget=64,
                   prefill_chunk=32, dp=dp, tp=tp)
comm = GlooCommunicator(r, tp, device_group)
if r == 0:
    llm = LLM(cfg, target=t, device="cpu", comm=comm, control=GroupAllGather(leaders), rank=g)
    loop = EngineLoop(llm.scheduler, channel=BroadcastChannel(host_group), rank=g, dp=llm.lockstep, idle_sleep=0.001)
else:
    llm = LLM(cfg, target=t, device="cpu", comm=comm)
    loop = EngineLoop(llm.scheduler, channel=BroadcastChannel(host_group), rank=r)
dist.barrier()
loop.start()
outs = []
if rank == 0:
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    tickets = [loop.submit([3 + i, 40 + i, 7, 9, 200 + i, 5] * (2 + i), sp) for i in range(4)]
    for tk in tickets:
        toks = []
        while True:
            kind, val = tk.events.get(timeout=120)
            if kind == "tokens":
                toks.extend(val)
            else:
                assert kind == "done", (kind, val)
                break
        outs.append(toks)
    loop.stop(timeout=60)
else:
    loop.thread.join(120)
with open(os.environ["HB_OUT"] + f".{rank}", "w") as f:
    json.dump({"outs": outs, "steps": loop.steps, "finished": llm.scheduler.metrics.finished,
               "healthy": loop.healthy, "alive": loop.thread.is_alive()}, f)
os._exit(0)
"""


def test_four_cpu_ranks_as_two_replicas_of_two_rank_groups(tmp_path):
    """The process groups of `replica_groups` (gloo here): world ranks 0-1 and 2-3 are the two replicas; rank 0 takes
    the requests, both replicas serve some, every follower takes its leader's steps, and stop ends all four."""
    script = tmp_path / "w.py"
    script.write_text(GROUPS_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HB_ROOT=root, HB_OUT=str(tmp_path / "out"))
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                        "--master-addr", "127.0.0.1", "--master-port", "29613", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    r = [json.loads((tmp_path / f"out.{i}").read_text()) for i in range(4)]
    assert len(r[0]["outs"]) == 4 and all(len(o) == 4 for o in r[0]["outs"])
    assert all(x["healthy"] and not x["alive"] for x in r)
    assert r[0]["finished"] + r[2]["finished"] == 4 and min(r[0]["finished"], r[2]["finished"]) >= 1
    assert r[1]["finished"] == r[0]["finished"] and r[3]["finished"] == r[2]["finished"]
    assert r[1]["steps"] == r[0]["steps"] and r[3]["steps"] == r[2]["steps"]
