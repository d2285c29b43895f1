"""Failure detection without faulting a GPU: a device wait that runs out returns a status the host reads, a
CommTimeout in a step fails every ticket and turns the API unhealthy, and a rank that stops answering between
steps is noticed through the store heartbeat so the supervisor restarts the group."""
import asyncio
import ctypes
import os
import sys
import time

import pytest
import torch

from hibana_b200 import _native as nv
from hibana_b200.parallel.watchdog import PeerWatchdog


class _DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_watchdog_reports_a_rank_that_stops_beating():
    store, now = _DictStore(), [0.0]
    clock = lambda: now[0]
    w0 = PeerWatchdog(store, 0, 3, timeout=5.0, clock=clock)
    w1 = PeerWatchdog(store, 1, 3, timeout=5.0, clock=clock)
    w2 = PeerWatchdog(store, 2, 3, timeout=5.0, clock=clock)
    for t in range(4):
        now[0] = float(t)
        for w in (w0, w1, w2):
            w.beat()
        assert w0.check() == [] and w1.check() == []
    for t in range(4, 12):          # rank 2 goes silent; rank 1 keeps beating
        now[0] = float(t)
        w0.beat()
        w1.beat()
        dead, dead1 = w0.check(), w1.check()
    assert dead == [2] and dead1 == [2]
    # a rank that never wrote a heartbeat counts from the watchdog's start
    w = PeerWatchdog(_DictStore(), 0, 2, timeout=1.0, clock=clock)
    now[0] += 2.0
    assert w.check() == [1]


WORKER = r"""
import os, sys, time
sys.path.insert(0, os.environ["HB_ROOT"])
import torch.distributed as dist
from hibana_b200.parallel.watchdog import PeerWatchdog
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
attempt_file = os.environ["HB_ATTEMPT"]
store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=__import__("datetime").timedelta(seconds=20))
if rank == 0:
    n = int(open(attempt_file).read() or 0) + 1 if os.path.exists(attempt_file) else 1
    open(attempt_file, "w").write(str(n))
    store.set("attempt", str(n))
attempt = int(store.get("attempt"))
def on_dead(ranks):
    open(os.environ["HB_LOG"], "a").write(f"rank {rank} attempt {attempt}: silent {list(ranks)}\n")
    os._exit(13)
store.set(f"ready/{rank}/{attempt}", "1")          # a slow import of another rank is not silence: start together
store.wait([f"ready/{r}/{attempt}" for r in range(world)])
wd = PeerWatchdog(store, rank, world, interval=0.05, timeout=2.5, on_dead=on_dead).start()
for step in range(120):           # the "engine steps" (6 s: a silent peer is noticed while they run)
    time.sleep(0.05)
    if attempt == 1 and rank == 1 and step == 3:
        wd.stop()                 # between steps: stops answering but stays alive (Popen.poll cannot see it)
        time.sleep(60)
store.set(f"done/{rank}", "1")
store.wait([f"done/{r}" for r in range(world)])
time.sleep(0.2)
os._exit(0)
"""


def test_silent_rank_is_detected_and_the_group_restarts(tmp_path):
    from hibana_b200.launch.supervisor import RankGroup, Supervisor
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HB_ROOT=root, HB_ATTEMPT=str(tmp_path / "attempt"), HB_LOG=str(tmp_path / "log"))
    group = RankGroup(2, [sys.executable, str(script)], master_port=29633, env=env)
    logs = []
    sup = Supervisor(group, log=logs.append)
    t0 = time.monotonic()
    rc = sup.run(poll_interval=0.05)
    # (a loaded machine can cost a further restart: a starved heartbeat thread, the store's port still closing;
    # what is checked is that the silent rank was seen, the group came back and finished)
    assert rc == 0 and len(sup.restarts) >= 1, logs
    assert time.monotonic() - t0 < 90
    log = (tmp_path / "log").read_text()
    assert "rank 0 attempt 1: silent [1]" in log
    assert int((tmp_path / "attempt").read_text()) >= 2


def test_comm_timeout_in_a_step_gives_503():
    """A bounded device wait that gave up surfaces as DeviceWaitTimeout from the step; the engine loop fails every
    ticket, later submissions are refused and /health turns 503."""
    import httpx
    from hibana_b200.api.server import create_app
    from hibana_b200.engine.loop import EngineLoop
    from hibana_b200.engine.scheduler import Scheduler, SchedulerConfig
    from hibana_b200.tokenizer import ByteTokenizer
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_scheduler import FakeExecutor

    class TimingOut(FakeExecutor):
        def decode_step(self, reqs):
            raise nv.DeviceWaitTimeout(4)

    loop = EngineLoop(Scheduler(TimingOut(), SchedulerConfig(max_batch=4))).start()
    app = create_app(loop, ByteTokenizer())

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t") as c:
            r = await c.post("/generate", json={"text": "abc", "sampling_params": {"max_new_tokens": 4}})
            assert r.status_code == 503 and "peer flag" in r.text
            assert (await c.get("/health")).status_code == 503
            assert (await c.post("/generate", json={"text": "abc"})).status_code == 503
    asyncio.run(go())
    assert not loop.healthy and "DeviceWaitTimeout" in loop.failure
    loop.stop()


def _heap(nbytes):
    out = ctypes.c_void_p()
    assert nv.lib().hb_comm_alloc(nbytes, ctypes.byref(out)) == 0
    return out.value


@pytest.mark.gpu
def test_device_wait_runs_out_and_the_context_stays_usable():
    """One process, one GPU: rank 0 of a 2-rank barrier whose "peer" is a second local heap that nobody serves.
    The flag never arrives, the wait gives up after its 2 ms limit, the kernel returns with kTimeoutPeer in the
    status word, the host raises; after the word is cleared and the peer's flag is published by hand the same
    call succeeds, and so does the fused all-reduce + norm on the same heaps."""
    from hibana_b200.parallel import comm as comm_mod  # registers the signatures
    dev = torch.device("cuda")
    lib = nv.lib()
    ctrl, nbytes = lib.hb_comm_ctrl_bytes(), lib.hb_comm_ctrl_bytes() + (1 << 20)
    mine, peer = _heap(nbytes), _heap(nbytes)
    bases = (ctypes.c_void_p * 2)(mine, peer)
    st = nv.device_state(dev)
    st.status.zero_()
    limit_ns = 2_000_000
    t0 = time.perf_counter()
    assert lib.hb_barrier(bases, 2, 0, 0, limit_ns, st.status.data_ptr(), nv.stream()) == 0
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert took < 1.0, took                       # the kernel came back by itself
    assert int(st.status[0]) == 4                 # kTimeoutPeer
    with pytest.raises(nv.DeviceWaitTimeout):
        c = comm_mod.Communicator.__new__(comm_mod.Communicator)
        c.device = dev
        c.check_status()
    assert int(st.status[0]) == 0                 # read_status cleared it
    # the peer "answers": flags[slot 0][src 1] of my control block reaches the sequence number being waited for
    heap = torch.as_tensor(comm_mod._RawCuda(mine, ctrl), device=dev).view(torch.int32)
    seq = int(heap[64 + 0].item())                # Ctrl.seq[0] follows flags[8][8]
    heap[0 * 8 + 1] = seq + 1
    torch.cuda.synchronize()
    assert lib.hb_barrier(bases, 2, 0, 0, limit_ns, st.status.data_ptr(), nv.stream()) == 0
    torch.cuda.synchronize()
    assert int(st.status[0]) == 0
    # fused all-reduce + residual + norm against the silent peer: times out, writes the status, returns
    rows, h = 4, 256
    res = torch.zeros(rows, h, dtype=torch.bfloat16, device=dev)
    w = torch.ones(h, dtype=torch.bfloat16, device=dev)
    out = torch.empty(rows, h, dtype=torch.bfloat16, device=dev)
    code = lib.hb_ar_norm(bases, 2, 0, 1, ctrl, rows, h, res.data_ptr(), w.data_ptr(), 1e-6, 0, out.data_ptr(), None,
                          None, None, 0, limit_ns, st.status.data_ptr(), -1, 0, nv.stream())
    assert code == 0
    torch.cuda.synchronize()
    assert nv.read_status(dev) == 4
    # and an ordinary kernel of the library still runs on the same context
    from hibana_b200.ops import basic
    x = torch.randn(8, 256, device=dev).bfloat16()
    y = basic.rmsnorm(x, w, 1e-6)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and nv.read_status(dev) == 0
    lib.hb_comm_free(ctypes.c_void_p(mine))
    lib.hb_comm_free(ctypes.c_void_p(peer))


@pytest.mark.gpu
def test_runner_raises_when_the_status_word_is_set():
    """The step's status read: a non-zero word copied back with the sampled tokens raises instead of returning them."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny
    model = DenseModel(dense_tiny(), "cuda:0", seed=0)
    ex = Executor(model, max_batch=2, max_ctx=128, use_graphs=False)
    ex.generate_batch([[1, 2, 3]], SamplingParams(max_tokens=2))
    nv.device_state(torch.device("cuda:0")).status[0] = 9
    with pytest.raises(nv.DeviceWaitTimeout):
        ex.generate_batch([[4, 5, 6]], SamplingParams(max_tokens=2))
    assert nv.read_status(torch.device("cuda:0")) == 0
    assert len(ex.generate_batch([[7, 8, 9]], SamplingParams(max_tokens=2))[0].output_ids) == 2


@pytest.mark.gpu
def test_checked_index_flavour_reports_a_bad_slot_and_skips_the_access(tmp_path):
    """The -DHB_BOUNDS build of the native library: a KV slot beyond the pool handed to the RoPE + KV-write kernel is
    recorded (kernel, index, limit) and nothing is written; valid calls report nothing and match the normal build.
    Runs in a child process because a process loads one flavour of the library."""
    import subprocess
    import sys
    script = tmp_path / "bounds_child.py"
    script.write_text('''
import json, os, sys, torch
sys.path.insert(0, os.environ["HB_ROOT"])
from hibana_b200 import config, _native as nv
config.install(config.EngineConfig(bounds=True))
from hibana_b200.cache.kv_pool import KvPool
from hibana_b200.ops import basic
assert nv.lib() is not None and nv.bounds_enabled(), "the checked flavour must be the one loaded before a bad index is tried"
dev = torch.device("cuda")
pool = KvPool(1, 64, 2, 128, torch.bfloat16, dev)
g = torch.Generator().manual_seed(0)
qkv = torch.randn(4, (4 + 2 * 2) * 128, generator=g).bfloat16().to(dev)
pos = torch.arange(4, dtype=torch.int32, device=dev)
inv = basic.rope_inv_freq(128, 1e6).to(dev)
good = torch.tensor([1, 2, 3, 4], dtype=torch.int32, device=dev)
basic.rope_kv_write(qkv, pos, good, inv, pool.k[0], pool.v[0], 4, 2, 128)
torch.cuda.synchronize()
clean = nv.read_bounds()
before = pool.storage.clone()
bad = torch.tensor([5, 70, 6, 7], dtype=torch.int32, device=dev)          # 70 > 64 slots + the dummy row
basic.rope_kv_write(qkv, pos, bad, inv, pool.k[0], pool.v[0], 4, 2, 128)
torch.cuda.synchronize()
rep = nv.read_bounds()
changed = (pool.storage != before).any(-1).any(0).any(0).any(0).nonzero().flatten().tolist()
print("RESULT " + json.dumps({"clean": clean, "report": rep, "changed_slots": changed, "again": nv.read_bounds(),
                              "status": nv.read_status(dev)}))
''')
    env = dict(os.environ, HB_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    proc = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    import json
    res = json.loads([l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["clean"] is None and res["again"] is None and res["status"] == 0
    assert res["report"] == {"hits": res["report"]["hits"], "kernel": "rope_kv_write", "index": 70, "limit": 65}
    assert res["changed_slots"] == [5, 6, 7]                 # the in-range rows were written, the bad one skipped
