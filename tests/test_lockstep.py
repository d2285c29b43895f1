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
