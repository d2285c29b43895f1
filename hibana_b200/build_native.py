"""Ahead-of-time build of the sm_100a native library.

One shared object, ``hibana_b200/lib/libhibana_b200.so``, holds every CUDA kernel and the C++ runtime pieces.
It is built in-tree with nvcc (``-gencode arch=compute_100a,code=sm_100a``; nvcc cross-compiles without a GPU)
and loaded with ctypes, so it needs no torch headers and compiles in seconds per file. The reference instead
JIT-compiles one torch extension per kernel at first use (hibana/kernels/w3.py:252,
hibana/engine/config.py:92).

Run ``python -m hibana_b200.build_native`` to (re)build; ``build()`` is incremental on file mtimes.
``build(bounds=True)`` (``--bounds``) makes the checked-index flavour ``libhibana_b200_bounds.so``: the same
sources with ``-DHB_BOUNDS -rdc=true``, in which every pool index a kernel is handed goes through a range check
that records the first violation and skips the access (csrc/hb_common.cuh ``index_ok``, csrc/bounds.cu).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ_DIR = CSRC / "build"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libhibana_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "-Xcudafe", "--diag_suppress=177",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread"]


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, nvcc: str, verbose: bool, extra: list[str], obj_dir: Path = OBJ_DIR) -> tuple[Path, str]:
    obj = obj_dir / (src.name + ".o")
    newest_dep = max(src.stat().st_mtime, _headers_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest_dep:
        return obj, ""
    if src.suffix == ".cu":
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cuda_inc = str(Path(nvcc).resolve().parent.parent / "include")
        cmd = ["g++", *CXX_FLAGS, "-I", str(CSRC), "-I", cuda_inc, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return obj, (proc.stderr if verbose else "")


BOUNDS_LIB_PATH = LIB_DIR / "libhibana_b200_bounds.so"


def build(verbose: bool = False, ptxas_info: bool = False, bounds: bool = False) -> Path:
    """Compiles what changed and links the library. Returns its path."""
    nvcc = nvcc_path()
    lib_path = BOUNDS_LIB_PATH if bounds else LIB_PATH
    obj_dir = CSRC / "build_bounds" if bounds else OBJ_DIR
    if nvcc is None:
        if lib_path.exists():
            return lib_path
        raise RuntimeError(f"nvcc not found and no prebuilt {lib_path.name}")
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    if bounds:
        extra += ["-DHB_BOUNDS", "-rdc=true"]      # one device-side record shared by every translation unit
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
        results = list(pool.map(lambda s: _compile(s, nvcc, verbose or ptxas_info, extra, obj_dir), srcs))
    objs = [o for o, _ in results]
    if verbose or ptxas_info:
        for _, log in results:
            if log:
                print(log, file=sys.stderr)
    newest_obj = max(o.stat().st_mtime for o in objs)
    if not lib_path.exists() or lib_path.stat().st_mtime < newest_obj:
        tmp = lib_path.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lpthread", *(["-rdc=true"] if bounds else [])]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, lib_path)
    return lib_path


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv, bounds="--bounds" in sys.argv)
    print(path)
