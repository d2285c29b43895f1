"""What `serve` checks and fetches before an engine starts: the host (CUDA devices of the right kind, free device
and host memory, the native library), the checkpoint the settings name (a local directory, or a pinned Hugging Face
snapshot looked up in the cache and downloaded when the hub is reachable), the calibrated 3-bit copies
(`<w3 root>/<target>-current`, the link the reference's launcher keeps), and a one-paragraph summary for the log.
Reference: hibana/launch/preflight.py:23-190 (check_host / snapshot_dir / download / ensure_snapshots / ensure_w3 /
summary) and hibana/target.py:249-285."""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

from ..hardware import b200

HEADROOM_BYTES = 20 << 30        # disk space a download leaves free


class PreflightError(RuntimeError):
    pass


def meminfo() -> dict:
    """/proc/meminfo in KiB ({} where the file does not exist)."""
    out = {}
    try:
        for line in Path("/proc/meminfo").read_text().splitlines():
            key, _, rest = line.partition(":")
            out[key] = int(rest.split()[0])
    except (OSError, ValueError, IndexError):
        pass
    return out


def snapshot_dir(cache: Path, repo: str, revision: str) -> Optional[Path]:
    """The complete snapshot of `repo` at `revision` under `cache` or `cache/hub` (Hugging Face cache layout):
    config.json and every weight file the index names are present. None when anything is missing."""
    for root in (Path(cache), Path(cache) / "hub"):
        d = root / f"models--{repo.replace('/', '--')}" / "snapshots" / revision
        index = d / "model.safetensors.index.json"
        try:
            files = set(json.loads(index.read_text())["weight_map"].values()) if index.is_file() else {"model.safetensors"}
        except (OSError, ValueError, KeyError):
            continue
        if (d / "config.json").is_file() and all((d / f).is_file() for f in files):
            return d
    return None


def download(cache: Path, repo: str, revision: str, log=print) -> Path:
    """Fetches one pinned snapshot into cache/hub after checking that it fits on the disk. Needs the hub client and
    a network; without them the error says what to copy where."""
    hub = Path(cache) / "hub"
    try:
        from huggingface_hub import HfApi, snapshot_download
    except ImportError as e:
        raise PreflightError(f"{repo}@{revision[:7]} is not in {cache} and huggingface_hub is not installed: copy the "
                             f"snapshot to {hub}/models--{repo.replace('/', '--')}/snapshots/{revision}") from e
    hub.mkdir(parents=True, exist_ok=True)
    os.environ["HF_HUB_OFFLINE"] = "0"
    try:
        info = HfApi().model_info(repo, revision=revision, files_metadata=True)
        snap = hub / f"models--{repo.replace('/', '--')}" / "snapshots" / revision
        missing = sum(s.size or 0 for s in info.siblings if not (snap / s.rfilename).is_file())
        free = shutil.disk_usage(hub).free
        if missing + HEADROOM_BYTES > free:
            raise PreflightError(f"{repo}@{revision[:7]} needs {missing / 1e9:.1f} GB more and {cache} has "
                                 f"{free / 1e9:.1f} GB free (keeping {HEADROOM_BYTES / 1e9:.0f} GB spare)")
        log(f"downloading {repo}@{revision[:7]} into {cache}: {missing / 1e9:.1f} GB")
        snapshot_download(repo, revision=revision, cache_dir=hub)
    except PreflightError:
        raise
    except Exception as e:  # noqa: BLE001 - no network, no such revision, ...
        raise PreflightError(f"could not fetch {repo}@{revision[:7]}: {type(e).__name__}: {e}") from e
    found = snapshot_dir(cache, repo, revision)
    if found is None:
        raise PreflightError(f"{repo}@{revision[:7]} is still incomplete in {cache} after the download")
    return found


def ensure_weights(cfg, cache: Optional[Path] = None, fetch: bool = True, log=print) -> Optional[Path]:
    """The checkpoint directory `cfg.weights` resolves to: None for random init, a local directory as it is, or
    `repo@revision` looked up in the cache (and downloaded when `fetch`)."""
    w = cfg.weights
    if not w or w == "random":
        return None
    if Path(w).is_dir():
        return Path(w)
    if "@" not in w:
        raise PreflightError(f"weights {w!r}: not a directory and not of the form repo@revision")
    repo, revision = w.split("@", 1)
    cache = Path(cache or os.environ.get("HF_HOME") or Path.home() / ".cache" / "huggingface")
    found = snapshot_dir(cache, repo, revision)
    if found is None and fetch:
        found = download(cache, repo, revision, log)
    if found is None:
        raise PreflightError(f"{repo}@{revision[:7]} is not in {cache}")
    return found


def ensure_w3(cfg, root: Optional[Path] = None, required: bool = False) -> Optional[Path]:
    """The calibrated 3-bit checkpoint to serve when `cfg.w3` is on: `<root>/<target>-current`, with its manifest and
    every file's checksum verified. None (3-bit copies are then made by nearest rounding at load) unless `required`."""
    if not cfg.w3:
        return None
    from ..weights import w3_reference
    root = Path(root or os.environ.get("HIBANA_W3_ROOT") or Path.home() / ".cache" / "hibana" / "w3-checkpoints")
    found = w3_reference.current_checkpoint(root, cfg.target)
    if found is None:
        if required:
            raise PreflightError(f"{cfg.target} serves calibrated 3-bit copies and {root}/{cfg.target}-current has none")
        return None
    try:
        w3_reference.ReferenceW3Checkpoint(found).verify()
    except (ValueError, OSError) as e:
        raise PreflightError(f"{found}: {e}") from e
    return found


def summary(cfg, host: "HostReport", weights: Optional[Path], w3: Optional[Path]) -> str:
    par = f"tp={cfg.tp}" + (f" dp={cfg.dp}" if cfg.dp > 1 else "") + (f" ep={cfg.ep}" if cfg.ep > 1 else "")
    spec = "off" if cfg.spec == "off" else f"{cfg.spec} depth {cfg.spec_depth}"
    mem = meminfo()
    lines = [f"target {cfg.target} ({cfg.profile}), {par}, weights {weights or 'random init'}",
             f"GPUs: {host.gpus} x {host.names[0] if host.names else '?'}; free "
             + ", ".join(f"{g:.0f}" for g in host.free_gib) + " GiB"
             + (f"; host {mem['MemAvailable'] // 2 ** 20} GiB available" if "MemAvailable" in mem else ""),
             f"batch {cfg.max_batch}, kv {cfg.kv_dtype or 'target default'}, state {cfg.ssm_state}, speculation {spec}, "
             f"graphs {'on' if cfg.cuda_graphs else 'off'}, radix cache {'on' if cfg.radix_cache else 'off'}"
             + (f", SSD tier {cfg.ssd_dir}" if cfg.ssd_dir else "")]
    if cfg.w3:
        lines.append(f"3-bit decode copies: {w3 or 'nearest-rounded at load'}")
    return "\n".join(lines)


@dataclass
class HostReport:
    ok: bool = True
    gpus: int = 0
    names: list = field(default_factory=list)
    problems: list = field(default_factory=list)
    free_gib: list = field(default_factory=list)


def check_host(need_gpus: int = 1, min_free_gib: float = 8.0, require_b200: bool = True) -> HostReport:
    rep = HostReport()
    try:
        import torch
    except ImportError:
        rep.ok = False
        rep.problems.append("torch is not importable")
        return rep
    if not torch.cuda.is_available():
        rep.ok = False
        rep.problems.append("no CUDA device")
        return rep
    rep.gpus = torch.cuda.device_count()
    if rep.gpus < need_gpus:
        rep.ok = False
        rep.problems.append(f"{need_gpus} GPUs needed, {rep.gpus} visible")
    for i in range(rep.gpus):
        p = torch.cuda.get_device_properties(i)
        rep.names.append(p.name)
        if require_b200 and not b200.is_target(p.major, p.minor):
            rep.ok = False
            rep.problems.append(f"GPU {i} is sm_{p.major}{p.minor} ({p.name}); the kernels are built for {b200.ARCH}")
        free, _ = torch.cuda.mem_get_info(i)
        rep.free_gib.append(free / (1 << 30))
        if free / (1 << 30) < min_free_gib:
            rep.ok = False
            rep.problems.append(f"GPU {i} has only {free / (1 << 30):.1f} GiB free")
    from .. import _native
    if not _native.LIB_PATH.exists():
        rep.ok = False
        rep.problems.append(f"{_native.LIB_PATH} missing: run python -m hibana_b200.build_native")
    return rep
