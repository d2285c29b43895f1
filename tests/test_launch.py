"""Settings resolution, supervisor restart policy, memory guard, traces, CLI parsing (all CPU, no processes)."""
import json
import signal

import pytest

from hibana_b200.cli import build_parser
from hibana_b200.config import EngineConfig, current, reset, using
from hibana_b200.engine.request import Request, SamplingParams
from hibana_b200.engine.traces import TraceSink, summarize
from hibana_b200.launch.guard import MemoryGuard
from hibana_b200.launch.settings import resolve
from hibana_b200.launch.supervisor import RankGroup, Supervisor


def test_resolution_order(tmp_path):
    f = tmp_path / "hibana.env"
    f.write_text("MAX_BATCH=16\nHIBANA_PORT=31000  # comment\n")
    cfg = resolve("dense", config_file=str(f), env={})
    assert cfg.target == "dense-27b" and cfg.max_batch == 16 and cfg.port == 31000
    cfg = resolve("dense", config_file=str(f), env={"HIBANA_MAX_BATCH": "32", "SHARAR_SEED": "7"})
    assert cfg.max_batch == 32 and cfg.seed == 7
    cfg = resolve("dense", config_file=str(f), env={"HIBANA_MAX_BATCH": "32"}, flags={"max_batch": 8})
    assert cfg.max_batch == 8
    assert resolve("tiny", env={}, profile="fast").accept_top_k == 2
    with pytest.raises(ValueError):
        resolve("dense", env={}, flags={"spec": "mtp"})           # no MTP head on the dense target
    with pytest.raises(ValueError):
        resolve("nope", env={})
    with pytest.raises(ValueError):
        EngineConfig(tp=3)


def test_config_context():
    reset()
    with using(EngineConfig(max_batch=5)) as c:
        assert current().max_batch == 5 and c.buckets == (1, 2, 4)
    assert EngineConfig().as_dict()["api_key"] == ""


class FakeProc:
    def __init__(self, codes):
        self.codes = codes          # sequence of poll() results
        self.signals = []

    def poll(self):
        return self.codes.pop(0) if len(self.codes) > 1 else self.codes[0]

    def send_signal(self, s):
        self.signals.append(s)
        self.codes = [0]

    def kill(self):
        self.codes = [-9]


def test_supervisor_restarts_then_gives_up():
    spawned = []

    def spawn(argv, env):
        # rank 1 of every generation dies right away with SIGKILL's code
        p = FakeProc([None, -9] if env["RANK"] == "1" else [None])
        spawned.append((env["RANK"], env["WORLD_SIZE"], env["MASTER_ADDR"]))
        return p
    clock = {"t": 0.0}
    sup = Supervisor(RankGroup(2, ["x"], spawn=spawn), clock=lambda: clock["t"],
                     sleep=lambda s: clock.__setitem__("t", clock["t"] + s), log=lambda m: None)
    assert sup.run(poll_interval=1.0) == 1
    assert len(spawned) == 2 * 6                       # first start + 5 restarts
    assert spawned[0] == ("0", "2", "127.0.0.1")


def test_supervisor_clean_exit():
    sup = Supervisor(RankGroup(2, ["x"], spawn=lambda argv, env: FakeProc([None, 0])), sleep=lambda s: None,
                     log=lambda m: None)
    assert sup.run() == 0


def test_memory_guard_fires_after_three_low_samples():
    sent = []
    vals = iter([10.0, 1.0, 1.0, 5.0, 1.0, 1.0, 1.0])
    g = MemoryGuard(8.0, pid=123, probe=lambda: next(vals), send=lambda pid, sig: sent.append((pid, sig)))
    fired = [g.sample() for _ in range(7)]
    assert fired == [False] * 6 + [True] and sent == [(123, signal.SIGTERM)]


def test_traces_roundtrip(tmp_path):
    sink = TraceSink(str(tmp_path))
    r = Request(prompt_ids=[1, 2, 3], params=SamplingParams(max_tokens=2))
    r.push(5)
    r.push(6)
    r.rounds = [2]
    sink.record(r)
    sink.close()
    s = summarize(str(tmp_path))
    assert s["requests"] == 1 and s["output_tokens"] == 2 and s["tokens_per_round"] == 2


def test_cli_parser():
    a = build_parser().parse_args(["serve", "27b", "--tp", "2", "--port", "30011", "--no-graphs"])
    assert a.cmd == "serve" and a.target == "27b" and a.tp == 2 and a.cuda_graphs is False
    a = build_parser().parse_args(["cache", "--flush"])
    assert a.flush


def test_preflight_snapshot_lookup_w3_link_and_summary(tmp_path):
    import json
    import torch
    from hibana_b200.config import EngineConfig
    from hibana_b200.launch import preflight as pf
    from hibana_b200.weights import w3_reference as ref
    from hibana_b200.weights.w3 import CodebookW3
    snap = tmp_path / "hub" / "models--org--model" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text("{}")
    (snap / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "m-1.safetensors"}}))
    assert pf.snapshot_dir(tmp_path, "org/model", "abc123") is None          # a weight file is missing
    (snap / "m-1.safetensors").write_bytes(b"x")
    assert pf.snapshot_dir(tmp_path, "org/model", "abc123") == snap
    cfg = EngineConfig(target="dense-tiny", weights="org/model@abc123")
    assert pf.ensure_weights(cfg, cache=tmp_path, fetch=False) == snap
    assert pf.ensure_weights(EngineConfig(target="dense-tiny"), cache=tmp_path) is None
    with pytest.raises(pf.PreflightError):
        pf.ensure_weights(cfg.replace(weights="org/other@ffff"), cache=tmp_path, fetch=False)
    with pytest.raises(pf.PreflightError):
        pf.ensure_weights(cfg.replace(weights="nowhere"), cache=tmp_path)
    # calibrated 3-bit copies: the <target>-current link, verified
    assert pf.ensure_w3(cfg.replace(w3=True), root=tmp_path) is None
    with pytest.raises(pf.PreflightError):
        pf.ensure_w3(cfg.replace(w3=True), root=tmp_path, required=True)
    w = CodebookW3.pack(torch.zeros(128, 128, dtype=torch.int64), torch.ones(128, 4).to(torch.float8_e4m3fn),
                        torch.ones(128), (-3.5, -2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 3.5))
    d = ref.write_directory(tmp_path / "calib", {"layers.0.mlp.down": w})
    (tmp_path / "dense-tiny-current").symlink_to(d)
    assert pf.ensure_w3(cfg.replace(w3=True), root=tmp_path) == d.resolve()
    assert pf.ensure_w3(cfg, root=tmp_path) is None                           # w3 off: nothing to look for
    host = pf.HostReport(gpus=8, names=["NVIDIA B200"] * 8, free_gib=[170.0] * 8)
    text = pf.summary(cfg.replace(w3=True, tp=8, spec="ngram"), host, snap, d)
    assert "tp=8" in text and "ngram depth" in text and str(d) in text
    assert isinstance(pf.meminfo(), dict)


def test_serve_flags_reach_the_settings():
    """Flags the docs name (`--w3 --w3-checkpoint`, `--ssm-state`, `--kv-dtype`, `--dp` with `--tp`) are parsed and
    land in the resolved settings; absent flags leave the defaults alone."""
    from hibana_b200 import cli
    ap = cli.build_parser()
    cfg = cli._resolve(ap.parse_args(["serve", "dense-tiny", "--w3", "--w3-checkpoint", "/ckpt/w3", "--ssm-state", "int8w",
                                      "--kv-dtype", "fp8", "--spec", "lilicorr", "--dp", "2", "--tp", "2"]))
    assert (cfg.w3, cfg.w3_checkpoint, cfg.ssm_state, cfg.kv_dtype, cfg.spec, cfg.dp, cfg.tp) == \
        (True, "/ckpt/w3", "int8w", "fp8", "lilicorr", 2, 2)
    plain = cli._resolve(ap.parse_args(["serve", "dense-tiny"]))
    assert plain.w3 is False and plain.ssm_state == "fp32" and plain.host_floor_gib == 6.0
