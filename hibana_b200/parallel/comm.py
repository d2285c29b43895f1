"""Communicator of one NVSwitch box: symmetric peer-mapped heap + fused collectives, NCCL as bootstrap/baseline.

One process per GPU. `Communicator.create` cudaMallocs this rank's heap, exchanges CUDA IPC handles over the
`torch.distributed` process group and maps every peer heap, after which the fused kernels in csrc/comm.cu reach
peer memory directly over NVLink. `all_reduce` (NCCL) is the baseline path; `slot_buffer` + `allreduce_norm` is
the fused path (the row-parallel GEMM writes its partial into a heap slot, then one kernel does all-reduce +
residual + RMSNorm (+ NVFP4 quantisation)). A CPU `FakeCommunicator` runs the same interface over gloo / in
process for tests. Reference: hibana/distributed.py:53-183.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import basic, nvfp4
from ..ops.nvfp4 import Nvfp4Tensor

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_comm_ctrl_bytes", [])
nv.register("hb_comm_nslot", [])
nv.register("hb_comm_alloc", [L, ctypes.POINTER(ctypes.c_void_p)])
nv.register("hb_comm_free", [P])
nv.register("hb_comm_ipc_handle", [P, P])
nv.register("hb_comm_ipc_open", [P, ctypes.POINTER(ctypes.c_void_p)])
nv.register("hb_comm_ipc_close", [P])
nv.register("hb_ar_norm", [P, I, I, I, L, I, I, P, P, Fl, I, P, P, P, P, I, L, P, L, I, P])
nv.register("hb_barrier", [P, I, I, I, L, P, P])
nv.register("hb_comm_sp_layout", [ctypes.POINTER(ctypes.c_longlong)])
nv.register("hb_rs_norm_ag", [P, I, I, I, I, L, I, P, P, Fl, I, L, L, L, P, I, L, P, P])
nv.register("hb_pick_exchange", [P, I, I, I, I, L, P, P, L, P, L, P, P])
nv.register("hb_gemm_peer", [I, P, P, P, P, I, I, I, P, L, P, I, P, I, I, I, L, L, L, L, L, P, I, I, P])


# Up to this many rows the push ("LL") protocol wins; above it the flag-based one-shot moves half the bytes.
LL_MAX_ROWS = 32


class _RawCuda:
    """Exposes a raw device pointer to torch through __cuda_array_interface__ (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


CommTimeout = nv.DeviceWaitTimeout     # raised by check_status and by the engine's per-step status read


class Communicator:
    def __init__(self, rank: int, world: int, device: torch.device, heap_ptr: int, heap_bytes: int, peer_ptrs: list,
                 slot_bytes: int, timeout_ms: int, group=None, fused: bool = True, sp_rows: int = 0,
                 sp_hidden: int = 0):
        self.rank, self.world, self.device = rank, world, device
        self.heap_ptr, self.heap_bytes, self.peer_ptrs = heap_ptr, heap_bytes, peer_ptrs
        self.slot_bytes = slot_bytes
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.group = group
        self.fused = fused
        self.nslot = nv.lib().hb_comm_nslot()
        self.ctrl_bytes = nv.lib().hb_comm_ctrl_bytes()
        self._bases = (ctypes.c_void_p * world)(*peer_ptrs)
        self.heap = torch.as_tensor(_RawCuda(heap_ptr, heap_bytes), device=device)
        self._next_slot = 0
        self._q_bufs: dict = {}
        # the push protocol (payload + sequence number in 8-byte words) wins on two ranks (12.5 vs 15.4 us for one row);
        # from four ranks on every rank lands world x the words and the one-shot flag protocol is faster (16 vs 36 us
        # at eight ranks), so it is the only one used there
        self.low_latency = world <= 2
        self.status = nv.device_state(device).status
        # sequence-parallel region: staging of scattered partials + gather buffers (NVFP4 and bf16)
        self.sp_rows, self.sp_hidden = sp_rows, sp_hidden
        if sp_rows:
            lay = (ctypes.c_longlong * 3)()
            nv.lib().hb_comm_sp_layout(lay)
            self.sp_cnt_off, self.sp_flag_off, self.sp_seq_off = int(lay[0]), int(lay[1]), int(lay[2])
            base = self.ctrl_bytes + self.nslot * slot_bytes
            self.sp_stage_off = base
            self.sp_bf_off = base + sp_rows * sp_hidden * 2
            self.sp_q_off = self.sp_bf_off + sp_rows * sp_hidden * 2
            self.sp_ka = nvfp4.k_atoms(sp_hidden)
            self.sp_sf_off = self.sp_q_off + sp_rows * sp_hidden // 2
            assert self.sp_sf_off + (sp_rows // 128 + 2) * self.sp_ka * 512 <= heap_bytes

    @classmethod
    def create(cls, rank: int, world: int, device: torch.device, *, slot_mb: int = 8, timeout_ms: int = 2000,
               group=None, fused: bool = True, sp_rows: int = 0, sp_hidden: int = 0) -> "Communicator":
        """Collective: every rank of `group` (default: the world group) must call it."""
        lib = nv.lib()
        torch.cuda.set_device(device)
        slot_bytes = slot_mb << 20
        heap_bytes = lib.hb_comm_ctrl_bytes() + lib.hb_comm_nslot() * slot_bytes
        if sp_rows:
            heap_bytes += sp_rows * sp_hidden * 5 + (sp_rows // 128 + 2) * nvfp4.k_atoms(sp_hidden) * 512 + 4096
        out = ctypes.c_void_p()
        nv.check(lib.hb_comm_alloc(heap_bytes, ctypes.byref(out)), "hb_comm_alloc", launches=0)
        handle = ctypes.create_string_buffer(64)
        nv.check(lib.hb_comm_ipc_handle(out, handle), "hb_comm_ipc_handle", launches=0)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        peers = []
        for r in range(world):
            if r == rank:
                peers.append(out.value)
            else:
                p = ctypes.c_void_p()
                nv.check(lib.hb_comm_ipc_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(p)),
                         "hb_comm_ipc_open", launches=0)
                peers.append(p.value)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        return cls(rank, world, device, out.value, heap_bytes, peers, slot_bytes, timeout_ms, group, fused, sp_rows,
                   sp_hidden)

    # ---- slots
    def slot_offset(self, slot: int) -> int:
        return self.ctrl_bytes + slot * self.slot_bytes

    def begin_forward(self, n_collectives: int) -> None:
        """Fixes the slot phase of a forward (or of the graph being captured): its collectives take slots
        0, 1, ... cyclically, and the cycle length is chosen so that the LAST collective of the forward never
        lands on the slot of the FIRST one. A slot's partial buffer (and its low-latency landing area) may be
        overwritten as soon as the owner has finished the collective, while a slow peer can still be reading it;
        what protects the peer is that every rank takes part in some other collective before the slot comes round
        again. Inside a forward that holds because consecutive collectives use different slots; across two
        forwards (replays of captured graphs in any order, slot ids baked in) it holds because every forward starts
        on slot 0 and never ends there. The last slot is reserved for `barrier`."""
        usable = self.nslot - 1
        self._cycle = next((c for c in (usable, usable - 1, usable - 2)
                            if n_collectives < 2 or (n_collectives - 1) % c != 0), usable)
        self._next_slot = 0
        self._single = n_collectives < 2

    def next_slot(self) -> int:
        """Slot of the next collective call site (the same order on every rank); see `begin_forward`."""
        s = self._next_slot
        cycle = getattr(self, "_cycle", self.nslot - 1)
        nxt = (s + 1) % cycle
        assert cycle < 2 or nxt != s
        if getattr(self, "_single", False):
            # a forward with one collective would reuse slot 0 back to back: a barrier separates the two uses
            self.barrier()
        self._next_slot = nxt
        return s

    def slot_buffer(self, slot: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        """A [rows, cols] tensor inside this rank's heap slot (what the producing GEMM writes into)."""
        nbytes = rows * cols * torch.tensor([], dtype=dtype).element_size()
        if nbytes > self.slot_bytes // 2:
            raise ValueError(f"message of {nbytes} bytes exceeds half of the {self.slot_bytes}-byte heap slot")
        off = self.slot_offset(slot)
        return self.heap[off:off + nbytes].view(dtype).view(rows, cols)

    def fits(self, rows: int, cols: int) -> bool:
        return self.fused and rows * cols * 2 <= self.slot_bytes // 2

    # ---- collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """NCCL all-reduce (sum), in place: the baseline path."""
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        """Gathers shards along the last dim (vocab-parallel logits)."""
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    PICK_ROWS = 4096      # row capacity of the greedy-pick landing area (16 bytes per row and rank)

    def pick_exchange(self, val: torch.Tensor, idx: torch.Tensor, idx_offset: int,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Vocab-parallel greedy token: `val` / `idx` [rows] are the best logit of this rank's vocabulary shard and
        its id inside the shard; returns the global id of the best over all ranks (identical on every rank).
        The landing area is the data region of the reserved barrier slot, which no other collective writes."""
        rows = val.shape[0]
        assert rows <= self.PICK_ROWS and self.world * self.PICK_ROWS * 16 <= self.slot_bytes
        out = torch.empty(rows, dtype=torch.int64, device=self.device) if out is None else out
        nv.check(nv.lib().hb_pick_exchange(self._bases, self.world, self.rank, rows, self.PICK_ROWS,
                                           self.slot_offset(self.nslot - 1), val.data_ptr(), idx.data_ptr(),
                                           idx_offset, out.data_ptr(), self.timeout_ns, self.status.data_ptr(),
                                           nv.stream()), "hb_pick_exchange")
        return out

    def allreduce_norm(self, slot: int, rows: int, h: int, *, residual: Optional[torch.Tensor],
                       weight: Optional[torch.Tensor], eps: float = 1e-6, gemma: bool = False,
                       quant_scale: Optional[torch.Tensor] = None, want_bf16: bool = True):
        """Fused one-shot all-reduce of the partial in `slot` + residual add + RMSNorm (+ NVFP4 quant).

        Returns (bf16 output or None, Nvfp4Tensor or None). `residual` is updated in place with sum + residual.
        """
        out = torch.empty(rows, h, dtype=torch.bfloat16, device=self.device) if want_bf16 else None
        q = sf = None
        ka = 0
        if quant_scale is not None:
            # persistent per-shape buffers: the padding scale rows are zeroed once, the kernel writes real rows only
            key = (rows, h)
            bufs = self._q_bufs.get(key)
            if bufs is None:
                q, sf = nvfp4._alloc(rows, h, self.device)
                sf.zero_()
                self._q_bufs[key] = (q, sf)
            else:
                q, sf = bufs
            ka = sf.shape[1]
        # small messages take the low-latency push protocol: the second half of the slot is its landing area
        ll_rows = (self.slot_bytes // 2) // (self.world * h * 4) if self.low_latency else 0
        ll_off = self.slot_offset(slot) + self.slot_bytes // 2 if (ll_rows >= rows and rows <= LL_MAX_ROWS) else -1
        nv.check(nv.lib().hb_ar_norm(self._bases, self.world, self.rank, slot, self.slot_offset(slot), rows, h,
                                     nv.ptr(residual), nv.ptr(weight), eps, int(gemma), nv.ptr(out), nv.ptr(q),
                                     nv.ptr(sf), nv.ptr(quant_scale), ka, self.timeout_ns, self.status.data_ptr(),
                                     ll_off, ll_rows, nv.stream()), "hb_ar_norm")
        xq = Nvfp4Tensor(q, sf, quant_scale, rows, h) if q is not None else None
        return out, xq

    # ---- sequence-parallel prefill chain (fused GEMM -> reduce-scatter, norm, all-gather -> GEMM)
    def sp_ok(self, rows: int, hidden: int) -> bool:
        return (self.fused and self.sp_rows >= rows and hidden == self.sp_hidden and rows % (128 * self.world) == 0)

    def sp_gemm_scatter(self, lin, x) -> None:
        """Row-parallel projection whose epilogue stores each partial tile into the owner rank's staging rows."""
        xq = x if isinstance(x, Nvfp4Tensor) or lin.fmt != "nvfp4" else lin.quantize_input(x)
        m = xq.rows if isinstance(xq, Nvfp4Tensor) else xq.shape[0]
        rpr = m // self.world
        if lin.fmt == "nvfp4":
            a, b, sfa, sfb, k, alpha, ka_a, ka_b = xq.q, lin.wq.q, xq.sf, lin.wq.sf, xq.k, lin.alpha, xq.ka, lin.wq.ka
            kind = 1
        else:
            a, b, sfa, sfb, k, alpha, ka_a, ka_b, kind = xq, lin.weight, None, None, xq.shape[1], None, 0, 0, 0
        nv.check(nv.lib().hb_gemm_peer(kind, a.data_ptr(), b.data_ptr(), nv.ptr(sfa), nv.ptr(sfb), m,
                                       lin.out_features, k, None, lin.out_features, nv.ptr(alpha), 4, self._bases,
                                       self.world, self.rank, rpr, self.sp_stage_off, self.sp_cnt_off, -1, 0,
                                       self.timeout_ns, self.status.data_ptr(), ka_a, ka_b, nv.stream()),
                 "hb_gemm_peer")

    def sp_reduce_norm_gather(self, rows: int, h: int, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                              gemma: bool = False, quant_scale: Optional[torch.Tensor] = None):
        """Owner rows: sum the staged partials, add the residual shard, RMSNorm, (quantise), push to every rank.
        Returns the full [rows, h] activation as it will appear in this rank's gather buffer (valid once the
        consumer's flag wait passes): an Nvfp4Tensor when `quant_scale` is given, else a bf16 tensor."""
        rpr = rows // self.world
        bn = 256 if h >= 256 else 128
        expected = (rpr // 128) * ((h + bn - 1) // bn)
        q_off = self.sp_q_off if quant_scale is not None else -1
        bf_off = -1 if quant_scale is not None else self.sp_bf_off
        nv.check(nv.lib().hb_rs_norm_ag(self._bases, self.world, self.rank, rpr, h, self.sp_stage_off, expected,
                                        residual.data_ptr(), weight.data_ptr(), eps, int(gemma), q_off, self.sp_sf_off,
                                        bf_off, nv.ptr(quant_scale), self.sp_ka, self.timeout_ns,
                                        self.status.data_ptr(), nv.stream()), "hb_rs_norm_ag")
        if quant_scale is not None:
            q = self.heap[self.sp_q_off:self.sp_q_off + rows * h // 2].view(rows, h // 2)
            nblk = (rows + 127) // 128
            sf = self.heap[self.sp_sf_off:self.sp_sf_off + nblk * self.sp_ka * 512].view(nblk, self.sp_ka, 512)
            return Nvfp4Tensor(q, sf, quant_scale, rows, h)
        return self.heap[self.sp_bf_off:self.sp_bf_off + rows * h * 2].view(torch.bfloat16).view(rows, h)

    def sp_gemm_gathered(self, lin, x, *, epilogue: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Column-parallel projection over gathered rows: each A row tile waits for its source rank's flag."""
        nvq = isinstance(x, Nvfp4Tensor)
        m = x.rows if nvq else x.shape[0]
        n = lin.out_features
        cols = n // 2 if epilogue == 2 else n
        out = torch.empty(m, cols, dtype=torch.bfloat16, device=self.device) if out is None else out
        if nvq:
            a, b, sfa, sfb, k, alpha, ka_a, ka_b, kind = x.q, lin.wq.q, x.sf, lin.wq.sf, x.k, lin.alpha, x.ka, lin.wq.ka, 1
        else:
            a, b, sfa, sfb, k, alpha, ka_a, ka_b, kind = x, lin.weight, None, None, x.shape[1], None, 0, 0, 0
        nv.check(nv.lib().hb_gemm_peer(kind, a.data_ptr(), b.data_ptr(), nv.ptr(sfa), nv.ptr(sfb), m, n, k,
                                       out.data_ptr(), out.stride(0), nv.ptr(alpha), epilogue, self._bases, self.world,
                                       self.rank, m // self.world, 0, 0, self.sp_flag_off, self.sp_seq_off,
                                       self.timeout_ns, self.status.data_ptr(), ka_a, ka_b, nv.stream()),
                 "hb_gemm_peer")
        return out

    def barrier(self, slot: Optional[int] = None) -> None:
        """Flag barrier on the reserved last slot (sequence-numbered, >= comparison: safe back to back)."""
        slot = self.nslot - 1 if slot is None else slot
        nv.check(nv.lib().hb_barrier(self._bases, self.world, self.rank, slot, self.timeout_ns,
                                     self.status.data_ptr(), nv.stream()), "hb_barrier")

    def check_status(self) -> None:
        """Host check at a publish point: raises CommTimeout when a bounded device wait gave up."""
        code = nv.read_status(self.device)
        if code:
            raise CommTimeout(code)

    # ---- host scalars (control plane)
    def min_int(self, v: int) -> int:
        t = torch.tensor([v], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return int(t.item())

    def max_float(self, v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def broadcast(self, obj=None, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, group_src=src, group=self.group)
        return box[0]


class FakeCommunicator:
    """Single-process stand-in with the Communicator interface over CPU tensors: holds every rank's partial so
    tests can play all ranks of a tensor-parallel model in one process (no GPU, no process group)."""

    def __init__(self, world: int):
        self.world, self.rank, self.fused = world, 0, False
        self.pending: list = []

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def fits(self, rows: int, cols: int) -> bool:
        return False

    def check_status(self) -> None:
        return None


class GlooCommunicator:
    """CPU ranks over a gloo process group: the host-side logic of tensor parallelism without a GPU."""

    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world, self.group, self.fused = rank, world, group, False

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        y = x.float()
        dist.all_reduce(y, group=self.group)
        x.copy_(y.to(x.dtype))
        return x

    def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def fits(self, rows: int, cols: int) -> bool:
        return False

    def min_int(self, v: int) -> int:
        t = torch.tensor([v], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return int(t.item())

    def max_float(self, v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def broadcast(self, obj=None, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, group_src=src, group=self.group)
        return box[0]

    def check_status(self) -> None:
        return None
