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


NVFP4 = "nvfp4"      # pool format: e2m1 values (two per byte) + one ue4m3 scale per 16 elements + a per-pool scale
NVFP4_KV_SCALE = 1.0 / 64.0


class KvPool:
    """`dtype` torch.bfloat16, torch.float8_e4m3fn or the string "nvfp4" (4.5 bits per element: K / V rows are
    quantised when they are written, csrc/misc.cu, and dequantised inside the attention kernel, csrc/attn.cu;
    reference: hibana/cache/kv_pool.py:24-66, hibana/kernels/kv_fp4.py:16-33)."""

    def __init__(self, layers: int, slots: int, kv_heads: int, head_dim: int, dtype=torch.bfloat16,
                 device: torch.device | str = "cpu", kv_scale: float = 1.0):
        self.layers, self.slots, self.kv_heads, self.head_dim = layers, slots, kv_heads, head_dim
        self.fp4 = dtype == NVFP4
        self.dtype, self.device = dtype, torch.device(device)
        self.kv_scale = NVFP4_KV_SCALE if self.fp4 and kv_scale == 1.0 else kv_scale
        # One allocation; slot 0 is the dummy row.
        if self.fp4:
            assert head_dim % 32 == 0
            self.storage = torch.zeros(max(layers, 1), 2, kv_heads, slots + 1, head_dim // 2, dtype=torch.uint8,
                                       device=device)
            self.sf = torch.zeros(max(layers, 1), 2, kv_heads, slots + 1, head_dim // 16, dtype=torch.uint8,
                                  device=device)
        else:
            self.storage = torch.zeros(max(layers, 1), 2, kv_heads, slots + 1, head_dim, dtype=dtype, device=device)
            self.sf = None
        self.k = [self.storage[i, 0].transpose(0, 1) for i in range(layers)]   # [slots + 1, kv_heads, head_dim]
        self.v = [self.storage[i, 1].transpose(0, 1) for i in range(layers)]
        if self.fp4:      # the scale rows travel with the value pools as an attribute the ops look for
            for i in range(layers):
                self.k[i].sf = self.sf[i, 0].transpose(0, 1)
                self.v[i].sf = self.sf[i, 1].transpose(0, 1)
        if self.device.type == "cuda":
            from .. import _native as nv
            nv.lib()
            nv.set_bound(nv.BOUND_KV_SLOTS, slots + 1)          # checked-index build: what a slot id may be
        # sparse-attention indexer pools (models/qsa.py): raw and compressed 128-wide index keys per slot and
        # attention layer, allocated by `enable_index` for targets that use the indexer on long contexts
        self.idx_raw: list = []
        self.idx_key: list = []
        self._free = list(range(slots, 0, -1))     # pop() hands out ascending ids (contiguous when fresh)
        self._owned = bytearray(slots + 1)
        self._shuffled = False                     # frees since the last sort

    def enable_index(self, layers: int, dim: int = 128) -> None:
        if not self.idx_raw:
            self.idx_raw = [torch.zeros(self.slots + 1, dim, dtype=torch.bfloat16, device=self.device)
                            for _ in range(layers)]
            self.idx_key = [torch.zeros(self.slots + 1, dim, dtype=torch.bfloat16, device=self.device)
                            for _ in range(layers)]

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def bytes_per_token(self) -> int:
        if self.fp4:
            return self.layers * 2 * self.kv_heads * (self.head_dim // 2 + self.head_dim // 16)
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
        if self.fp4:      # two regions of the payload: all value rows, then all scale rows
            cut = n * self.layers * 2 * self.kv_heads * (self.head_dim // 2)
            flat = payload.view(torch.uint8).view(-1)
            self._copy_region(self.storage, ids, flat[:cut], to_pool)
            self._copy_region(self.sf, ids, flat[cut:cut + n * self.layers * 2 * self.kv_heads * (self.head_dim // 16)],
                              to_pool)
            return
        self._copy_region(self.storage, ids, payload, to_pool)

    def _copy_region(self, storage: torch.Tensor, ids: torch.Tensor, payload: torch.Tensor, to_pool: bool) -> None:
        n = ids.numel()
        width = storage.shape[-1]
        if storage.is_cuda:
            from .. import _native as nv
            nv.register("hb_kv_copy", [nv.P, nv.P, nv.P, nv.I, nv.I, nv.I, nv.L, nv.I, nv.I, nv.I, nv.P])
            nv.check(nv.lib().hb_kv_copy(storage.data_ptr(), payload.data_ptr(), ids.data_ptr(), n,
                                         storage.shape[0], self.kv_heads, self.slots + 1, width,
                                         storage.element_size(), int(to_pool), nv.stream()), "hb_kv_copy")
            return
        view = payload.view(storage.dtype).view(n, storage.shape[0], 2, self.kv_heads, width)
        idx = ids.long()
        if to_pool:
            storage[:, :, :, idx] = view.permute(1, 2, 3, 0, 4)
        else:
            view.copy_(storage[:, :, :, idx].permute(3, 0, 1, 2, 4))

    def rows(self, ids: list[int]) -> torch.Tensor:
        """All layers' K and V rows of the given slots: [layers, 2, len(ids), kv_heads, head_dim] (a copy; for an
        NVFP4 pool the packed values and the scale bytes side by side along the last dim)."""
        idx = torch.tensor(ids, dtype=torch.long, device=self.device)
        out = self.storage[:, :, :, idx].transpose(2, 3).contiguous()
        if self.fp4:
            out = torch.cat((out, self.sf[:, :, :, idx].transpose(2, 3)), dim=-1)
        return out

    def dequantized(self, layer: int, which: int, ids: list[int]) -> torch.Tensor:
        """fp32 rows [len(ids), kv_heads, head_dim] of K (which = 0) or V (1) as attention sees them."""
        idx = torch.tensor(ids, dtype=torch.long, device=self.device)
        pool = (self.k if which == 0 else self.v)[layer]
        return dequant_rows(pool[idx], getattr(pool, "sf", None)[idx] if self.fp4 else None, self.kv_scale)

    def write_rows(self, ids: list[int], rows: torch.Tensor) -> None:
        idx = torch.tensor(ids, dtype=torch.long, device=self.device)
        self.storage[:, :, :, idx] = rows.to(self.storage.dtype).transpose(2, 3)


def dequant_rows(vals: torch.Tensor, sf, kv_scale: float) -> torch.Tensor:
    """Pool rows [..., D] (bf16 / e4m3) or packed NVFP4 rows [..., D / 2] with scales [..., D / 16] -> fp32 [..., D]."""
    if sf is None:
        return vals.float() * (kv_scale if vals.dtype != torch.bfloat16 else 1.0)
    from ..ops import nvfp4
    shape = vals.shape[:-1]
    flat = nvfp4.dequantize_ref(vals.reshape(-1, vals.shape[-1]), sf.reshape(-1, sf.shape[-1]), kv_scale)
    return flat.view(*shape, vals.shape[-1] * 2)
