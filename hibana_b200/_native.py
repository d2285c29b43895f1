"""ctypes loader of ``lib/libhibana_b200.so`` and thin call helpers.

The library is loaded once per process. On a machine with a CUDA device a missing library is an error (the
kernels are the product; there is no silent PyTorch fallback on GPU). On a CPU-only machine ``lib()`` returns
``None`` and the ops fall back to their plain-PyTorch reference implementations, which is what the CPU test
suite exercises.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_TRIED = False
_LOCK = threading.Lock()
LIB_PATH = Path(__file__).resolve().parent / "lib" / "libhibana_b200.so"
BOUNDS_LIB_PATH = LIB_PATH.with_name("libhibana_b200_bounds.so")

P, I, L, F = c_void_p, c_int, c_longlong, c_float

# name -> argtypes (all functions return int unless listed in _VOID)
_SIGS: dict[str, list] = {
    "hb_gemm": [I, P, P, P, P, I, I, I, L, L, P, L, P, F, P, I, I, I, P, P, P, I, I, I, P],
    "hb_quant_nvfp4": [P, L, I, I, I, P, P, P, I, P],
    "hb_norm_quant_nvfp4": [P, P, P, F, I, I, I, I, P, P, P, P, P],
    "hb_quant_fp8_static": [P, L, P, P, P],
    "hb_quant_fp8_rows": [P, I, I, P, P, P],
}
_VOID = {"hb_clear_tmap_cache": []}


def register(name: str, argtypes: list, void: bool = False) -> None:
    """Lets op modules declare the signature of the exports they call."""
    (_VOID if void else _SIGS)[name] = argtypes
    if _LIB is not None:
        _bind(_LIB, name, argtypes, void)


def _bind(lib: ctypes.CDLL, name: str, argtypes: list, void: bool) -> None:
    try:
        fn = getattr(lib, name)
    except AttributeError:
        return
    fn.argtypes = argtypes
    fn.restype = None if void else c_int


def lib() -> Optional[ctypes.CDLL]:
    global _LIB, _TRIED
    if _LIB is not None or _TRIED:
        return _LIB
    with _LOCK:
        if _LIB is not None or _TRIED:
            return _LIB
        _TRIED = True
        from . import config
        bounds = config.current().bounds       # the checked-index flavour (build_native.build(bounds=True))
        path = BOUNDS_LIB_PATH if bounds else LIB_PATH
        if not path.exists():
            try:
                from . import build_native

                build_native.build(bounds=bounds)
            except Exception:  # noqa: BLE001 - reported below when a GPU is present
                pass
        if path.exists() and torch.cuda.is_available():
            loaded = ctypes.CDLL(str(path))
            for name, sig in _SIGS.items():
                _bind(loaded, name, sig, False)
            for name, sig in _VOID.items():
                _bind(loaded, name, sig, True)
            _LIB = loaded
        elif torch.cuda.is_available():
            raise RuntimeError(
                f"{path} is missing on a machine with a CUDA device; run `python -m hibana_b200.build_native`")
    return _LIB


BOUND_KV_SLOTS, BOUND_STATE_SLOTS, BOUND_VOCAB, BOUND_ROWS = 0, 1, 2, 3
BOUND_KERNELS = {1: "rope_kv_write", 2: "kv_copy", 3: "conv1d", 4: "mamba2_scan", 5: "gdn_scan", 6: "attn_decode",
                 7: "attn_general", 8: "embedding"}


def bounds_enabled() -> bool:
    """True when the loaded library is the checked-index flavour."""
    loaded = lib()
    return bool(loaded is not None and hasattr(loaded, "hb_bounds_enabled") and loaded.hb_bounds_enabled())


def set_bound(which: int, value: int) -> None:
    """Tells the checked-index flavour the size of a pool (no-op in the normal build). Pools call it when built."""
    if _LIB is not None and bounds_enabled():
        _LIB.hb_bounds_set.argtypes = [c_int, c_longlong]
        check(_LIB.hb_bounds_set(which, int(value)), "hb_bounds_set", launches=0)


def read_bounds() -> Optional[dict]:
    """The first out-of-range index a kernel was handed since the last read ({"hits", "kernel", "index", "limit"}),
    or None; the access itself was skipped. Always None in the normal build."""
    if not bounds_enabled():
        return None
    out = (c_longlong * 4)()
    torch.cuda.synchronize()
    check(_LIB.hb_bounds_read(out), "hb_bounds_read", launches=0)
    if not out[0]:
        return None
    return {"hits": int(out[0]), "kernel": BOUND_KERNELS.get(int(out[1]), str(out[1])), "index": int(out[2]),
            "limit": int(out[3])}


def available() -> bool:
    return lib() is not None


def use_native(*tensors: torch.Tensor) -> bool:
    """True when the op should run the CUDA kernel: every tensor is on a CUDA device (and the library loads)."""
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    if lib() is None:
        raise RuntimeError("CUDA tensors given but the native library is not loaded")
    return True


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


CALLS = 0      # native entry points called
LAUNCHES = 0   # kernels those calls launched (each call launches at least one)


def check(code: int, what: str, launches: int = 1) -> None:
    global CALLS, LAUNCHES
    CALLS += 1
    LAUNCHES += launches
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


class _DeviceState:
    """Per-device scratch the kernels share: status word, split-K workspace and self-resetting counters."""

    def __init__(self, device: torch.device):
        self.status = torch.zeros(8, dtype=torch.int32, device=device)
        self.workspaces: dict[int, torch.Tensor] = {}
        self.counters: dict[int, torch.Tensor] = {}
        self.device = device

    def workspace(self, nbytes: int) -> tuple[torch.Tensor, torch.Tensor]:
        key = stream()
        ws = self.workspaces.get(key)
        if ws is None or ws.numel() * 4 < nbytes:
            size = max(nbytes, WORKSPACE_BYTES)
            ws = torch.empty(size // 4, dtype=torch.float32, device=self.device)
            self.workspaces[key] = ws
        cnt = self.counters.get(key)
        if cnt is None:
            cnt = torch.zeros(4096, dtype=torch.int32, device=self.device)
            self.counters[key] = cnt
        return ws, cnt


WORKSPACE_BYTES = 64 << 20
_STATES: dict[int, _DeviceState] = {}


def device_state(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATES.get(idx)
    if st is None:
        st = _DeviceState(torch.device("cuda", idx))
        _STATES[idx] = st
    return st


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (peer flag, arrival counter, mbarrier) gave up; the step's results are void."""

    def __init__(self, code: int):
        super().__init__(f"device-side wait ran out (status {code}: {STATUS_NAMES.get(code, 'unknown')})")
        self.code = code


STATUS_NAMES = {1: "tma stage never arrived", 2: "no free stage", 3: "accumulator never completed",
                4: "peer flag", 5: "arrival counter", 6: "bad shape", 7: "drain", 8: "low-latency word",
                9: "gated tile never saw its rows", 10: "expert-parallel receive buffer overflow"}


def read_status(device: Optional[torch.device] = None) -> int:
    """Reads (and clears) the device status word; non-zero means a bounded wait gave up (see hb_common.cuh)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = device_state(device)
    code = int(st.status[0].item())
    if code:
        st.status.zero_()
    return code
