"""Detached start of a server process with a pid file and a log under $HIBANA_RESULTS/logs.
Reference: hibana/launch/service.py (systemd-run detach); here a plain double-fork-free subprocess."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

from .ctl import pid_file


def log_path(name: str) -> Path:
    root = Path(os.environ.get("HIBANA_RESULTS", str(Path.home() / ".cache" / "hibana")))
    p = root / "logs" / f"{name}.log"
    p.parent.mkdir(parents=True, exist_ok=True)
    return p


def launch_detached(argv: list[str], port: int, name: str = "serve") -> int:
    log = open(log_path(f"{name}-{port}"), "ab")
    proc = subprocess.Popen([sys.executable, "-m", "hibana_b200", *argv], stdout=log, stderr=subprocess.STDOUT,
                            start_new_session=True)
    f = pid_file(port)
    f.parent.mkdir(parents=True, exist_ok=True)
    f.write_text(str(proc.pid))
    return proc.pid
