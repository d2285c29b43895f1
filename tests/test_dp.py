from hibana_b200.engine.dp import ReplicaSet, lockstep_plan


class _Loop:
    def __init__(self):
        self.n = 0
        self.got = []

    def submit(self, req):
        self.n += 1
        self.got.append(req)
        return len(self.got)

    def stats(self):
        return {"running": self.n, "waiting": 0}


class _Req:
    def __init__(self, ids):
        self.prompt_ids = ids


def test_least_loaded_routing_and_prefix_affinity():
    loops = [_Loop(), _Loop(), _Loop()]
    rs = ReplicaSet(loops, affinity_tokens=4, affinity_slack=2)
    for i in range(6):
        rs.submit(_Req([i, 1, 2]))                       # short prompts: pure least-loaded
    assert [l.n for l in loops] == [2, 2, 2]
    conv = list(range(100, 110))
    rs.submit(_Req(conv))
    home = max(range(3), key=lambda i: loops[i].n)
    loops[(home + 1) % 3].n = 1                          # another replica becomes a bit idler...
    rs.submit(_Req(conv + [7, 8]))
    assert loops[home].n == 4                            # ...but the conversation stays with its cached prefix
    loops[home].n = 50                                   # far busier: affinity gives way
    rs.submit(_Req(conv + [9]))
    assert loops[home].n == 50
    st = rs.stats()
    assert st["replicas"] == 3 and sum(st["routed"]) == 9


def test_lockstep_plan():
    assert lockstep_plan([False, False]) == (False, [False, False])
    assert lockstep_plan([True, False, True]) == (True, [False, True, False])


def test_lockstep_rounds_align_forwards_not_steps():
    """Three ranks with different amounts of work: every round has all ranks in it, a rank without a forward of
    its own learns that a peer has one, messages travel with the rounds, and everyone leaves in the same round."""
    import threading
    from hibana_b200.engine.dp import FORWARD, LEAVING, RUNNING, Lockstep, ThreadAllGather
    tg = ThreadAllGather(3, timeout=20)
    work = [3, 1, 0]                                 # forwards each rank wants
    log = [[] for _ in range(3)]
    mail = [[] for _ in range(3)]

    def run(rank):
        ls = Lockstep(tg.view(rank), rank, 3)
        ls.on_items = lambda src, items: mail[rank].extend((src, i) for i in items)
        if rank == 0:
            ls.post(("hello", 7))
        left = work[rank]
        while True:
            states = ls.round(FORWARD if left else LEAVING)
            log[rank].append(tuple(states))
            if left:
                left -= 1
            if all(s == LEAVING for s in states):
                break
    th = [threading.Thread(target=run, args=(r,)) for r in range(3)]
    for t in th:
        t.start()
    for t in th:
        t.join(30)
    assert log[0] == log[1] == log[2]
    assert [s.count(FORWARD) for s in log[0]] == [2, 1, 1, 0] and RUNNING not in log[0][0]
    assert mail[1] == [(0, ("hello", 7))] and mail[2] == [(0, ("hello", 7))] and mail[0] == []


def test_data_parallel_replicas_with_expert_parallel_layers_match_one_process():
    """Two replicas (threads, CPU), each holding half of every MoE layer's experts and serving its own prompts
    (different numbers, lengths and output lengths, one replica idle at the end) produce the tokens one process
    with all experts produces."""
    import threading
    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.dp import ThreadAllGather
    from hibana_b200.engine.llm import LLM
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.target import scaled, tiny_hybrid_moe
    t = scaled(tiny_hybrid_moe(), mtp_layers=0, mtp_depth=0)
    base = EngineConfig(target="tiny", max_batch=4, cuda_graphs=False, max_context=256, prefill_budget=64,
                        prefill_chunk=32)
    prompts = [[[5, 9, 11, 300, 17] * 9, [7, 8, 9]], [[100 + i for i in range(50)]]]
    params = [[SamplingParams(max_tokens=6, ignore_eos=True), SamplingParams(max_tokens=3, ignore_eos=True)],
              [SamplingParams(max_tokens=11, ignore_eos=True)]]
    one = LLM(base, target=t, device="cpu")
    want = [[r.output_ids for r in one.generate(prompts[i], params[i])] for i in range(2)]
    tg = ThreadAllGather(2, timeout=120)
    got, errs, llms = [None, None], [], [None, None]

    def run(rank):
        try:
            llm = LLM(base.replace(dp=2, ep=2), target=t, device="cpu", control=tg.view(rank), rank=rank)
            llms[rank] = llm
            got[rank] = [r.output_ids for r in llm.generate(prompts[rank], params[rank])]
        except Exception as e:   # noqa: BLE001 - reported by the assertion below
            errs.append(repr(e))
            tg.barrier.abort()
    th = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for x in th:
        x.start()
    for x in th:
        x.join(300)
    assert not errs, errs
    assert got == want
    ls0, ls1 = llms[0].lockstep, llms[1].lockstep
    assert ls0.rounds == ls1.rounds and ls0.empty_forwards + ls1.empty_forwards > 0
    assert llms[0].ep.calls == llms[1].ep.calls            # every rank ran every MoE all-to-all
    assert llms[0].model.blocks[0].ffn.experts.experts == t.experts // 2


def test_engine_loops_of_two_replicas_route_requests_and_stream_back_to_rank0():
    """Rank 0 owns the inbox: it gives every request an owner, the owner generates, tokens come back to rank 0's
    tickets with the rounds, and `stop` ends both loops in the same round."""
    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.dp import ThreadAllGather
    from hibana_b200.engine.llm import LLM
    from hibana_b200.engine.loop import EngineLoop
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.target import scaled, tiny_hybrid_moe
    t = scaled(tiny_hybrid_moe(), mtp_layers=0, mtp_depth=0)
    base = EngineConfig(target="tiny", max_batch=4, cuda_graphs=False, max_context=256, prefill_budget=64,
                        prefill_chunk=32)
    prompts = [[3 + i, 40 + i, 7, 9, 200 + i, 5] * (2 + i) for i in range(5)]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    want = [r.output_ids for r in LLM(base, target=t, device="cpu").generate(prompts, sp)]
    tg = ThreadAllGather(2, timeout=120)
    llms = [LLM(base.replace(dp=2, ep=2), target=t, device="cpu", control=tg.view(r), rank=r) for r in range(2)]
    loops = [EngineLoop(llms[r].scheduler, rank=r, dp=llms[r].lockstep, idle_sleep=0.001).start() for r in range(2)]
    tickets = [loops[0].submit(p, sp) for p in prompts]
    got = []
    for tk in tickets:
        toks = []
        while True:
            kind, val = tk.events.get(timeout=120)
            if kind == "tokens":
                toks += val
            else:
                assert kind == "done", (kind, val)
                break
        got.append(toks)
    assert got == want
    served = [llms[r].scheduler.metrics.finished for r in range(2)]
    assert sum(served) == 5 and min(served) >= 1, served
    assert loops[0]._router.loops[0].n == 0 and loops[0]._router.loops[1].n == 0
    loops[0].stop(timeout=30)
    loops[1].thread.join(30)
    assert not loops[0].thread.is_alive() and not loops[1].thread.is_alive()
    assert loops[0].healthy and loops[1].healthy


def test_replicas_of_tensor_parallel_groups_route_follow_and_stop():
    """dp = 2 replicas, each a tp = 2 group (four engine threads): rank 0 of replica 0 owns the inbox and routes;
    each group's leader joins the replicas' rounds and its follower applies the commands the leader broadcasts, so
    both ranks of a group take the same steps; tokens come back to rank 0's tickets; `stop` ends all four loops."""
    import threading

    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.dp import ThreadAllGather
    from hibana_b200.engine.llm import LLM
    from hibana_b200.engine.loop import EngineLoop
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.parallel.lockstep import ThreadBroadcast
    from hibana_b200.target import dense_tiny, scaled
    from test_tp import ThreadComm
    t = scaled(dense_tiny(), weight_format="bf16")
    base = EngineConfig(target="dense-tiny", max_batch=4, cuda_graphs=False, max_context=128, prefill_budget=64,
                        prefill_chunk=32)
    prompts = [[3 + i, 40 + i, 7, 9, 200 + i, 5] * (2 + i) for i in range(6)]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    want = [r.output_ids for r in LLM(base, target=t, device="cpu").generate(prompts, sp)]
    cfg = base.replace(dp=2, tp=2)
    leaders = ThreadAllGather(2, timeout=120)
    comms = [ThreadComm(2), ThreadComm(2)]
    chans = [ThreadBroadcast(2, timeout=120), ThreadBroadcast(2, timeout=120)]
    llms, loops, errs = {}, {}, []
    built = threading.Barrier(5)

    def rank_main(g, r):
        try:
            view = comms[g].view(r)
            view.rank = r
            if r == 0:
                llm = LLM(cfg, target=t, device="cpu", comm=view, control=leaders.view(g), rank=g)
                loop = EngineLoop(llm.scheduler, channel=chans[g].view(0), rank=g, dp=llm.lockstep, idle_sleep=0.001)
            else:
                llm = LLM(cfg, target=t, device="cpu", comm=view)
                assert llm.lockstep is None
                loop = EngineLoop(llm.scheduler, channel=chans[g].view(r), rank=r)
            llms[g, r], loops[g, r] = llm, loop
            built.wait(120)
            loop.start()
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))
            built.abort()

    threads = [threading.Thread(target=rank_main, args=(g, r)) for g in range(2) for r in range(2)]
    for th in threads:
        th.start()
    built.wait(120)
    for th in threads:
        th.join(60)
    assert not errs, errs
    assert llms[0, 0].model.target.tp_size == 2 and llms[1, 1].model.target.tp_rank == 1
    tickets = [loops[0, 0].submit(p, sp) for p in prompts]
    got = []
    for tk in tickets:
        toks = []
        while True:
            kind, val = tk.events.get(timeout=120)
            if kind == "tokens":
                toks += val
            else:
                assert kind == "done", (kind, val)
                break
        got.append(toks)
    assert all(len(g_) == 5 for g_ in got)
    assert sum(a[0] == b[0] for a, b in zip(got, want)) == len(want)      # reassociation only: first tokens match tp = 1
    served = [llms[g, 0].scheduler.metrics.finished for g in range(2)]
    assert sum(served) == 6 and min(served) >= 1, served
    loops[0, 0].stop(timeout=60)
    for key, loop in loops.items():
        loop.thread.join(60)
        assert not loop.thread.is_alive(), key
        assert loop.healthy, (key, loop.failure)
    for g in range(2):     # a follower took exactly its leader's steps
        assert llms[g, 1].scheduler.metrics.finished == served[g]
        assert llms[g, 1].executor.stats["decode_steps"] == llms[g, 0].executor.stats["decode_steps"]
        assert loops[g, 1].steps == loops[g, 0].steps


def test_a_failing_replica_leader_takes_its_follower_and_the_other_replicas_down():
    """Failure on the host inside a replica that is a tensor-parallel group: the leader of replica 1 raises in a
    step; it tells its follower (command channel) and the other replicas (next round); every loop ends unhealthy and
    rank 0's open tickets get the error instead of hanging."""
    import threading

    from hibana_b200.config import EngineConfig
    from hibana_b200.engine.dp import ThreadAllGather
    from hibana_b200.engine.llm import LLM
    from hibana_b200.engine.loop import EngineLoop
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.parallel.lockstep import ThreadBroadcast
    from hibana_b200.target import dense_tiny, scaled
    from test_tp import ThreadComm
    t = scaled(dense_tiny(), weight_format="bf16")
    cfg = EngineConfig(target="dense-tiny", max_batch=4, cuda_graphs=False, max_context=128, prefill_budget=64,
                       prefill_chunk=32, dp=2, tp=2)
    leaders = ThreadAllGather(2, timeout=20)
    comms = [ThreadComm(2), ThreadComm(2)]
    for c in comms:       # a collective nobody joins ends with an error, as a process-group timeout would
        c.barrier = threading.Barrier(2, timeout=10)
    chans = [ThreadBroadcast(2, timeout=20), ThreadBroadcast(2, timeout=20)]
    llms, loops = {}, {}
    for g in range(2):
        for r in range(2):
            view = comms[g].view(r)
            view.rank = r
            if r == 0:
                llms[g, r] = LLM(cfg, target=t, device="cpu", comm=view, control=leaders.view(g), rank=g)
                loops[g, r] = EngineLoop(llms[g, r].scheduler, channel=chans[g].view(0), rank=g, dp=llms[g, r].lockstep,
                                         idle_sleep=0.001)
            else:
                llms[g, r] = LLM(cfg, target=t, device="cpu", comm=view)
                loops[g, r] = EngineLoop(llms[g, r].scheduler, channel=chans[g].view(r), rank=r)

    def boom():
        raise RuntimeError("injected step failure")
    llms[1, 0].scheduler.step = boom              # replica 1's leader fails before its forward starts
    for loop in loops.values():
        loop.start()
    sp = SamplingParams(max_tokens=50, ignore_eos=True)
    tickets = [loops[0, 0].submit([3 + i, 40 + i, 7, 9, 200 + i, 5] * 3, sp) for i in range(4)]
    for loop in loops.values():
        loop.thread.join(60)
        assert not loop.thread.is_alive()
    assert not any(loop.healthy for loop in loops.values())
    assert "injected step failure" in loops[1, 0].failure
    # replica 1's follower had started the step its leader never joined: its collective gave up, or the leader's
    # message reached it first
    assert "leader failed" in loops[1, 1].failure or "Barrier" in loops[1, 1].failure
    assert "replica 1 failed" in loops[0, 0].failure and "leader failed" in loops[0, 1].failure
    for tk in tickets:
        last = None
        while not tk.events.empty():
            last = tk.events.get_nowait()
        assert last is not None and last[0] == "error", last
