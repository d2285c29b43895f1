"""Token-granular paged KV pool.

One row ("slot") per cached token and attention layer: k, v [layers][slots, kv_heads, head_dim] in bf16 or
e4m3. Physically the pool is head-major ([kv_heads, slots, head_dim]; the tensors handed out are strided views):
an attention CTA walks one kv head, so the tokens of a run of consecutive slots are one contiguous stream and
travel as bulk tensor copies with full DRAM page locality. Slots are handed out in ascending runs and freed
slots are re-sorted before large allocations, so sequences keep such runs. Slot 0 is a dummy that padded graph
rows read and write. The pool only allocates and frees; ownership
and `committed_len` belong to the StateManager. Reference: hibana/cache/kv_pool.py:24-139 (page size 1, free
list, pad pages, `write`).
"""
from __future__ import annotations

from typing import Iterable

import torch


class KvPool:
    def __init__(self, layers: int, slots: int, kv_heads: int, head_dim: int, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str = "cpu", kv_scale: float = 1.0):
        self.layers, self.slots, self.kv_heads, self.head_dim = layers, slots, kv_heads, head_dim
        self.dtype, self.device, self.kv_scale = dtype, torch.device(device), kv_scale
        # One allocation; slot 0 is the dummy row.
        self.storage = torch.zeros(max(layers, 1), 2, kv_heads, slots + 1, head_dim, dtype=dtype, device=device)
        self.k = [self.storage[i, 0].transpose(0, 1) for i in range(layers)]   # [slots + 1, kv_heads, head_dim]
        self.v = [self.storage[i, 1].transpose(0, 1) for i in range(layers)]
        self._free = list(range(slots, 0, -1))     # pop() hands out ascending ids (contiguous when fresh)
        self._owned = bytearray(slots + 1)
        self._shuffled = False                     # frees since the last sort

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def bytes_per_token(self) -> int:
        return self.layers * 2 * self.kv_heads * self.head_dim * self.storage.element_size()

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise MemoryError(f"KV pool exhausted: need {n}, free {len(self._free)}")
        if self._shuffled and n >= 32:
            self._free.sort(reverse=True)          # a prefill-sized request gets ascending runs again
            self._shuffled = False
        out = [self._free.pop() for _ in range(n)]
        for s in out:
            self._owned[s] = 1
        return out

    def free(self, ids: Iterable[int]) -> None:
        for s in ids:
            if s <= 0 or s > self.slots or not self._owned[s]:
                raise ValueError(f"double free or foreign slot {s}")
            self._owned[s] = 0
            self._free.append(s)
            self._shuffled = True

    def check(self) -> None:
        assert len(set(self._free)) == len(self._free), "duplicate free slots"
        assert all(not self._owned[s] for s in self._free)
        assert sum(self._owned) + len(self._free) == self.slots

    def copy_payload(self, ids: torch.Tensor, payload: torch.Tensor, to_pool: bool) -> None:
        """Moves the rows of slots `ids` (int32, on the pool's device) of all layers between the pool and a linear
        payload [len(ids), layers * 2 * kv_heads * head_dim] (device or pinned host memory): one kernel launch on
        CUDA (csrc/kv_copy.cu), indexing on CPU."""
        n = ids.numel()
        if n == 0:
            return
        if self.storage.is_cuda:
            from .. import _native as nv
            nv.register("hb_kv_copy", [nv.P, nv.P, nv.P, nv.I, nv.I, nv.I, nv.L, nv.I, nv.I, nv.I, nv.P])
            nv.check(nv.lib().hb_kv_copy(self.storage.data_ptr(), payload.data_ptr(), ids.data_ptr(), n,
                                         self.storage.shape[0], self.kv_heads, self.slots + 1, self.head_dim,
                                         self.storage.element_size(), int(to_pool), nv.stream()), "hb_kv_copy")
            return
        view = payload.view(self.storage.dtype).view(n, self.storage.shape[0], 2, self.kv_heads, self.head_dim)
        idx = ids.long()
        if to_pool:
            self.storage[:, :, :, idx] = view.permute(1, 2, 3, 0, 4)
        else:
            view.copy_(self.storage[:, :, :, idx].permute(3, 0, 1, 2, 4))

    def rows(self, ids: list[int]) -> torch.Tensor:
        """All layers' K and V rows of the given slots: [layers, 2, len(ids), kv_heads, head_dim] (a copy)."""
        idx = torch.tensor(ids, dtype=torch.long, device=self.device)
        return self.storage[:, :, :, idx].transpose(2, 3).contiguous()

    def write_rows(self, ids: list[int], rows: torch.Tensor) -> None:
        idx = torch.tensor(ids, dtype=torch.long, device=self.device)
        self.storage[:, :, :, idx] = rows.to(self.storage.dtype).transpose(2, 3)
