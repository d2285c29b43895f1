"""Recurrent-state pool: one slot per running sequence or cached snapshot.

Per recurrent layer a slot holds the causal-conv window (last conv_width - 1 raw rows, bf16) and the SSM /
delta-rule state (fp32; fp16 with stochastic rounding or int8 windows as options). Slot 0 is the dummy row padded
graph rows use. Reference: hibana/cache/state_pool.py:25-103 (`conv_all`, `ssm_all`, `copy_slot`).
"""
from __future__ import annotations

import torch


class StatePool:
    def __init__(self, layers: int, slots: int, conv_dim: int, conv_width: int, state_shape: tuple,
                 device: torch.device | str = "cpu", state_dtype: torch.dtype = torch.float32, window: int = 0,
                 groups: int = 1):
        """`window` > 0 (with int8 states of shape [heads, P, N]): the window-record format of ops/ssm_window.py:
        the int8 tensor is the boundary state and every slot also holds up to window + 16 committed-token records
        (B per group, dt * x and the running decay per head)."""
        self.layers, self.slots = layers, slots
        self.device = torch.device(device)
        self.conv = torch.zeros(max(layers, 1), slots + 1, conv_dim, max(conv_width - 1, 1), dtype=torch.bfloat16,
                                device=device)
        self.ssm = torch.zeros(max(layers, 1), slots + 1, *state_shape, dtype=state_dtype, device=device)
        # int8 states carry one fp32 scale per state row (last dim is the quantised one)
        self.ssm_scale = (torch.ones(max(layers, 1), slots + 1, *state_shape[:-1], dtype=torch.float32, device=device)
                          if state_dtype == torch.int8 else None)
        self.window = window if state_dtype == torch.int8 else 0
        self._records: list = []
        if self.window:
            h, p, n = state_shape
            cap = self.window + 16
            nl = max(layers, 1)
            self.win_b = torch.zeros(nl, slots + 1, groups, cap, n, dtype=torch.float16, device=device)
            self.win_u = torch.zeros(nl, slots + 1, h, cap, p, dtype=torch.float16, device=device)
            self.win_c = torch.zeros(nl, slots + 1, h, cap, dtype=torch.float32, device=device)
            self.win_len = torch.zeros(nl, slots + 1, groups, dtype=torch.int32, device=device)
            self._records = [self.win_b, self.win_u, self.win_c, self.win_len]
        if self.device.type == "cuda":
            from .. import _native as nv
            nv.lib()
            nv.set_bound(nv.BOUND_STATE_SLOTS, slots + 1)       # checked-index build: what a state slot may be
        # auxiliary per-slot state of layers that are not recurrences proper (the per-layer-embedding layer's
        # convolution window and token history): copied, cleared and snapshotted with the slot
        self.aux: dict = {}
        self._aux_fill: dict = {}
        self._free = list(range(slots, 0, -1))
        self._owned = bytearray(slots + 1)
        self.reserved = 0               # slots held for good by engine parts (captured rounds' scratch), not requests

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def bytes_per_slot(self) -> int:
        scale = self.ssm_scale[:, 0].numel() * 4 if self.ssm_scale is not None else 0
        aux = sum(a[0].numel() * a.element_size() for a in self.aux.values())
        aux += sum(r[:, 0].numel() * r.element_size() for r in self._records)
        return self.conv[:, 0].numel() * 2 + self.ssm[:, 0].numel() * self.ssm.element_size() + scale + aux

    def window_state(self, layer: int):
        """Layer `layer`'s view of the window records (ops/ssm_window.py `WindowState`)."""
        from ..ops.ssm_window import WindowState
        return WindowState(self.ssm[layer], self.ssm_scale[layer], self.win_b[layer], self.win_u[layer],
                           self.win_c[layer], self.win_len[layer], self.window)

    def register_aux(self, name: str, shape: tuple, dtype: torch.dtype, fill=0) -> torch.Tensor:
        """A [slots + 1, *shape] tensor that lives and moves with the slots (idempotent per name). Reference:
        hibana/cache/state_pool.py `register_aux`."""
        if name not in self.aux:
            self.aux[name] = torch.full((self.slots + 1, *shape), fill, dtype=dtype, device=self.device)
            self._aux_fill[name] = fill
        return self.aux[name]

    def alloc(self) -> int:
        if not self._free:
            raise MemoryError("state pool exhausted")
        s = self._free.pop()
        self._owned[s] = 1
        return s

    def reserve(self, n: int) -> list:
        """Takes `n` slots for the life of the pool (scratch of captured speculative rounds)."""
        out = [self.alloc() for _ in range(n)]
        self.reserved += n
        return out

    def free(self, slot: int) -> None:
        if slot <= 0:
            return
        if not self._owned[slot]:
            raise ValueError(f"double free of state slot {slot}")
        self._owned[slot] = 0
        self._free.append(slot)

    def copy_slot(self, src: int, dst: int) -> None:
        self.conv[:, dst].copy_(self.conv[:, src])
        self.ssm[:, dst].copy_(self.ssm[:, src])
        if self.ssm_scale is not None:
            self.ssm_scale[:, dst].copy_(self.ssm_scale[:, src])
        for a in self.aux.values():
            a[dst].copy_(a[src])
        for r in self._records:
            r[:, dst].copy_(r[:, src])

    def zero_slot(self, slot: int) -> None:
        self.conv[:, slot].zero_()
        self.ssm[:, slot].zero_()
        if self.ssm_scale is not None:
            self.ssm_scale[:, slot].fill_(1.0)
        for name, a in self.aux.items():
            a[slot].fill_(self._aux_fill[name])
        for r in self._records:
            r[:, slot].zero_()

    def export_slot(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        return self.conv[:, slot].clone(), self.ssm[:, slot].clone()

    def import_slot(self, slot: int, conv: torch.Tensor, ssm: torch.Tensor) -> None:
        self.conv[:, slot].copy_(conv)
        self.ssm[:, slot].copy_(ssm)

    def check(self) -> None:
        assert len(set(self._free)) == len(self._free)
        assert sum(self._owned) + len(self._free) == self.slots
