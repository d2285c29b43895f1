"""Host checks before an engine starts: CUDA device kind, driver, free memory, native library.
Reference: hibana/launch/preflight.py (check_host / download / ensure_w3) and hibana/target.py:249-285."""
from __future__ import annotations

from dataclasses import dataclass, field


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
        if require_b200 and (p.major, p.minor) != (10, 0):
            rep.ok = False
            rep.problems.append(f"GPU {i} is sm_{p.major}{p.minor} ({p.name}); the kernels are built for sm_100a")
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
