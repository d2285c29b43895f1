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
