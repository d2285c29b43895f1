"""Side-stream branches: independent launches of one layer run beside each other.

Small-batch decode is bound by the fixed cost of its kernels, not by bytes: two chains that do not depend on each
other (a MoE layer's shared expert beside its routed experts, the latent down-projection beside the router) cost
their sum on one stream and their maximum on two. `Branch` forks a side stream off the current one with an event,
runs what is launched inside `with branch:` there, and `join()` makes the current stream wait for it. Inside a CUDA
graph capture the fork and the join become graph edges, so the captured step keeps the two chains parallel; in eager
mode the tensors handed to `join` are recorded on the consuming stream (the caching allocator must not reuse them
while the side stream still owns them). Native launches pick the stream up through `_native.stream()`, and the
per-stream workspaces / counters of `_native._DeviceState` keep the two chains from sharing scratch.
"""
from __future__ import annotations

from typing import Optional

import torch

_SIDE: dict = {}


def side_stream(device: torch.device, index: int = 0) -> "torch.cuda.Stream":
    key = (device.index if device.index is not None else torch.cuda.current_device(), index)
    s = _SIDE.get(key)
    if s is None:
        s = _SIDE[key] = torch.cuda.Stream(device=device)
    return s


class Branch:
    """with Branch(x) as b: y = f(x)   # runs on the side stream, after everything queued so far
       ...                            # the current stream goes on meanwhile
       b.join(y)                      # the current stream waits for the branch; y is safe to use from here"""

    def __init__(self, like: torch.Tensor, enabled: bool = True, index: int = 0):
        self.enabled = enabled and like.is_cuda
        self._ctx = None
        if self.enabled:
            self.main = torch.cuda.current_stream(like.device)
            self.side = side_stream(like.device, index)
            self._done: Optional[torch.cuda.Event] = None

    def __enter__(self) -> "Branch":
        if self.enabled:
            fork = torch.cuda.Event()
            fork.record(self.main)
            self.side.wait_event(fork)
            self._ctx = torch.cuda.stream(self.side)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc) -> None:
        if self.enabled:
            self._done = torch.cuda.Event()
            self._done.record(self.side)
            self._ctx.__exit__(*exc)

    def mark(self) -> Optional["torch.cuda.Event"]:
        """An event at this point of the branch (inside `with`): `wait(event)` later joins up to here only."""
        if not self.enabled:
            return None
        ev = torch.cuda.Event()
        ev.record(self.side)
        return ev

    def wait(self, event, *tensors: torch.Tensor) -> None:
        if self.enabled and event is not None:
            self.main.wait_event(event)
            for t in tensors:
                if t is not None:
                    t.record_stream(self.main)

    def join(self, *tensors: torch.Tensor) -> None:
        self.wait(getattr(self, "_done", None), *tensors)
