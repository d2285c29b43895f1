"""Expert parallelism with an all-to-all over NVLink peer memory (csrc/ep.cu + the expert-parallel modes of the
grouped GEMM in csrc/gemm.cu).

Every rank keeps `experts / world` consecutive experts and routes its OWN tokens (attention ran data- or
sequence-parallel). `ExpertParallel.forward` is one mixture-of-experts call: count -> plan -> dispatch (rows
pushed straight into the owners' receive buffers, NVFP4-quantised once at the source) -> grouped fc1 gated on the
senders' flags -> activation (+ requantisation) -> grouped fc2 whose epilogue stores every result row into the
return buffer of the rank it came from -> combine gated on the owners' flags (top-k weighted sum + shared expert).
`forward_nccl` is the library-collective counterpart (all-gather of the tokens, local experts over all of them,
reduce-scatter of the partial sums) used as baseline and oracle. The reference has no all-to-all expert
parallelism; its two-rank mode replicates activations (hibana/model/flashnext/moe.py:68-192,
hibana/kernels/csrc/w3_gemm.cu `namespace moe`).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops import basic, gemm, moe, nvfp4
from .comm import _RawCuda

P, I, L, Fl = nv.P, nv.I, nv.L, nv.F
nv.register("hb_ep_ctrl_bytes", [])
nv.register("hb_ep_ctrl_layout", [P], void=True)
nv.register("hb_ep_count", [P, I, I, P, I, I, L, P])
nv.register("hb_ep_plan", [P, I, I, P, I, I, L, I, P, P, P, P, P, L, P, P])
nv.register("hb_ep_dispatch", [P, L, I, I, I, I, P, P, P, P, I, I, L, L, L, L, P])
nv.register("hb_ep_combine", [P, P, P, L, P, L, I, I, I, P, I, I, L, L, P, P])
nv.register("hb_gemm_grouped_ep", [I, P, P, P, P, I, I, I, I, P, L, P, I, P, P, I, P, I, I, P, I, I, P, P, P, L, P, L,
                                   L, I, P, P, I, P])
nv.register("hb_moe_tiles", [P, I, I, P, P, I, P])

EPI_RETURN = 5


def _align(v: int, a: int = 1024) -> int:
    return (v + a - 1) // a * a


class ExpertParallel:
    """Symmetric heap + kernel sequence of the expert-parallel all-to-all. Collective: all ranks call `create`
    and every `forward` together (a rank without tokens passes an empty batch)."""

    def __init__(self, rank, world, device, heap_ptr, heap_bytes, peer_ptrs, layout, *, tokens, topk, experts, hidden,
                 hidden_out, fmt, rows_cap, timeout_ms, group):
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self.heap_ptr, self.heap_bytes, self.peer_ptrs = heap_ptr, heap_bytes, peer_ptrs
        self.tokens, self.topk, self.experts, self.hidden, self.hidden_out = tokens, topk, experts, hidden, hidden_out
        self.fmt, self.rows_cap = fmt, rows_cap
        self.e_per = experts // world
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self._bases = (ctypes.c_void_p * world)(*peer_ptrs)
        self.heap = torch.as_tensor(_RawCuda(heap_ptr, heap_bytes), device=device)
        self.off = layout
        lay = (ctypes.c_longlong * 4)()
        nv.lib().hb_ep_ctrl_layout(lay)
        self.flag_rows_off, self.flag_ret_off, self.seq_off, self.done_fc2_off = (int(v) for v in lay)
        self.status = nv.device_state(device).status
        dev = device
        self.grp_cnt = torch.zeros(self.e_per, dtype=torch.int32, device=dev)
        self.grp_start = torch.zeros(self.e_per, dtype=torch.int32, device=dev)
        self.total_rows = torch.zeros(1, dtype=torch.int32, device=dev)
        self.dst_rank = torch.empty(max(tokens * topk, 1), dtype=torch.int32, device=dev)
        self.dst_row = torch.empty(max(tokens * topk, 1), dtype=torch.int32, device=dev)
        self.ka = nvfp4.k_atoms(hidden)

    # ---- construction
    @staticmethod
    def plan_layout(world, tokens, topk, experts, hidden, hidden_out, fmt, rows_cap) -> tuple[dict, int]:
        off, cur = {}, _align(nv.lib().hb_ep_ctrl_bytes())
        for name, nbytes in (("cnt_mat", world * experts * 4), ("row_ret", rows_cap * 4),
                             ("recv_q", rows_cap * hidden // 2 if fmt == "nvfp4" else 0),
                             ("recv_sf", (rows_cap // 128 + 1) * nvfp4.k_atoms(hidden) * 512 if fmt == "nvfp4" else 0),
                             ("recv_bf", rows_cap * hidden * 2 if fmt != "nvfp4" else 0),
                             ("ret", max(tokens * topk, 1) * hidden_out * 2)):
            off[name] = cur
            cur = _align(cur + nbytes)
        return off, cur

    @classmethod
    def create(cls, rank: int, world: int, device: torch.device, *, tokens: int, topk: int, experts: int, hidden: int,
               hidden_out: Optional[int] = None, fmt: str = "nvfp4", rows_cap: Optional[int] = None,
               timeout_ms: int = 2000, group=None) -> "ExpertParallel":
        """`tokens` bounds the tokens of one rank per call; `rows_cap` the rows one rank can receive (default: the
        worst case, every pair of every rank)."""
        assert experts % world == 0 and world <= 8
        lib = nv.lib()
        torch.cuda.set_device(device)
        hidden_out = hidden if hidden_out is None else hidden_out
        e_per = experts // world
        if rows_cap is None:
            rows_cap = (world * tokens * topk + 127) // 128 * 128 + min(e_per, world * tokens * topk) * 128
        layout, heap_bytes = cls.plan_layout(world, tokens, topk, experts, hidden, hidden_out, fmt, rows_cap)
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
        return cls(rank, world, device, out.value, heap_bytes, peers, layout, tokens=tokens, topk=topk,
                   experts=experts, hidden=hidden, hidden_out=hidden_out, fmt=fmt, rows_cap=rows_cap,
                   timeout_ms=timeout_ms, group=group)

    # ---- views into this rank's heap
    def _view(self, name: str, nbytes: int) -> torch.Tensor:
        o = self.off[name]
        return self.heap[o:o + nbytes]

    def _ptr(self, byte_off: int) -> int:
        return self.heap_ptr + byte_off

    # ---- one mixture-of-experts call
    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: "moe.ExpertWeights", *,
                shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, H] bf16 (this rank's tokens), ids int32 [T, k] GLOBAL expert ids, weights fp32 [T, k]; `ew` holds
        this rank's experts [rank * e_per, (rank + 1) * e_per). Returns [T, H_out] bf16."""
        lib, dev, st = nv.lib(), self.device, self.status
        t = x.shape[0]
        assert t <= self.tokens and ids.shape[1] == self.topk and ew.experts == self.e_per and ew.fmt == self.fmt
        h, h_out, rows_cap = self.hidden, self.hidden_out, self.rows_cap
        pairs = t * self.topk
        stream = nv.stream()
        nv.check(lib.hb_ep_count(nv.ptr(ids) if t else None, pairs, self.experts, self._bases, self.world, self.rank,
                                 self.off["cnt_mat"], stream), "hb_ep_count")
        nv.check(lib.hb_ep_plan(nv.ptr(ids) if t else None, pairs, self.experts, self._bases, self.world, self.rank,
                                self.off["cnt_mat"], rows_cap, self.grp_cnt.data_ptr(), self.grp_start.data_ptr(),
                                self.total_rows.data_ptr(), self.dst_rank.data_ptr(), self.dst_row.data_ptr(),
                                self.timeout_ns, st.data_ptr(), stream), "hb_ep_plan")
        nvq = self.fmt == "nvfp4"
        nv.check(lib.hb_ep_dispatch(nv.ptr(x) if t else None, x.stride(0) if t else h, t, self.topk, h, self.ka,
                                    self.dst_rank.data_ptr(), self.dst_row.data_ptr(),
                                    ew.fc1_in_scale.data_ptr() if nvq else None, self._bases, self.world, self.rank,
                                    self.off["recv_q"], self.off["recv_sf"], self.off["recv_bf"], self.off["row_ret"],
                                    stream), "hb_ep_dispatch")
        n1 = ew.n1
        epi1 = gemm.EPI_SILU_MUL if ew.act == "swiglu" else gemm.EPI_STORE
        h1 = torch.empty(rows_cap, ew.inter if ew.act == "swiglu" else n1, dtype=torch.bfloat16, device=dev)
        max_rows = min(self.world * self.tokens, rows_cap)
        # every rank sends about as many pairs as it has: expected rows per local expert
        bn_hint = moe.tile_hint(max(pairs, 1) , self.e_per, max_rows, self.fmt)
        bn_full = 16
        while bn_full < max_rows and bn_full < 256:
            bn_full *= 2
        bn_hint = min(bn_hint, bn_full)
        # compact (expert, chunk) work list from the planned row counts: the GEMM grids cover tiles that have rows
        # at most one partial tile per local expert beside the full ones of every pair that can arrive here
        tile_cap = -(-(self.world * self.tokens * self.topk) // bn_hint) + self.e_per
        tiles = torch.empty(tile_cap, dtype=torch.int32, device=dev)
        n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        nv.check(lib.hb_moe_tiles(self.grp_cnt.data_ptr(), self.e_per, bn_hint, tiles.data_ptr(), n_tiles.data_ptr(),
                                  tile_cap, stream), "hb_moe_tiles")
        gate = self._ptr(self.flag_rows_off)
        seq = self._ptr(self.seq_off)

        def grouped(kind, a, b, sfa, sfb, n_per, k, out, ldo, alpha, epi, ka_a, ka_b, *, gate_flags, ret):
            nv.check(lib.hb_gemm_grouped_ep(
                kind, a, b, sfa, sfb, self.e_per, n_per, rows_cap, k, out, ldo, alpha, epi, self.grp_start.data_ptr(),
                self.grp_cnt.data_ptr(), max_rows, st.data_ptr(), ka_a, ka_b, self._bases, self.world, self.rank,
                gate_flags, seq, self._ptr(self.off["row_ret"]) if ret else None, self.off["ret"],
                self._ptr(self.done_fc2_off) if ret else None, self.flag_ret_off, self.timeout_ns, bn_hint,
                tiles.data_ptr(), n_tiles.data_ptr(), tile_cap, stream),
                "hb_gemm_grouped_ep")

        if nvq:
            sf_rows = rows_cap // 128 + 1
            grouped(1, ew.fc1.q.data_ptr(), self._ptr(self.off["recv_q"]), ew.fc1.sf.data_ptr(),
                    self._ptr(self.off["recv_sf"]), n1, h, h1.data_ptr(), h1.stride(0), ew.fc1_alpha.data_ptr(), epi1,
                    ew.fc1.ka, self.ka, gate_flags=gate, ret=False)
            mid = basic.act_mul(h1, basic.ACT_RELU2) if ew.act == "relu2" else h1
            q2, sf2 = nvfp4._alloc(rows_cap, ew.inter, dev)
            nv.check(lib.hb_quant_nvfp4_rows(mid.data_ptr(), mid.stride(0), rows_cap, ew.inter, sf2.shape[1],
                                             ew.fc2_in_scale.data_ptr(), q2.data_ptr(), sf2.data_ptr(), 0, None,
                                             self.total_rows.data_ptr(), stream), "hb_quant_nvfp4_rows")
            grouped(1, ew.fc2.q.data_ptr(), q2.data_ptr(), ew.fc2.sf.data_ptr(), sf2.data_ptr(), h_out, ew.inter,
                    None, h_out, ew.fc2_alpha.data_ptr(), EPI_RETURN, ew.fc2.ka, sf2.shape[1], gate_flags=None,
                    ret=True)
            del sf_rows
        else:
            grouped(0, ew.fc1.data_ptr(), self._ptr(self.off["recv_bf"]), None, None, n1, h, h1.data_ptr(),
                    h1.stride(0), None, epi1, 0, 0, gate_flags=gate, ret=False)
            mid = basic.act_mul(h1, basic.ACT_RELU2) if ew.act == "relu2" else h1
            grouped(0, ew.fc2.data_ptr(), mid.data_ptr(), None, None, h_out, ew.inter, None, h_out, None, EPI_RETURN,
                    0, 0, gate_flags=None, ret=True)
        out = torch.empty(t, h_out, dtype=torch.bfloat16, device=dev)
        nv.check(lib.hb_ep_combine(nv.ptr(weights) if t else None, self.dst_rank.data_ptr(), nv.ptr(shared),
                                   shared.stride(0) if shared is not None else 0, nv.ptr(out) if t else None,
                                   out.stride(0) if t else h_out, t, self.topk, h_out, self._bases, self.world,
                                   self.rank, self.off["ret"], self.timeout_ns, st.data_ptr(), stream),
                 "hb_ep_combine")
        return out

    # ---- NCCL-only counterpart (baseline / oracle)
    def forward_nccl(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: "moe.ExpertWeights", *,
                     shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Same result through library collectives: all-gather the tokens (padded to `tokens` per rank), run the
        local experts over all of them, reduce-scatter the partial sums."""
        t, cap = x.shape[0], self.tokens
        dev = self.device

        def padded(v, fill=0):
            out = torch.full((cap,) + tuple(v.shape[1:]), fill, dtype=v.dtype, device=dev)
            out[:t] = v
            return out

        xs = torch.empty(self.world * cap, self.hidden, dtype=x.dtype, device=dev)
        idg = torch.empty(self.world * cap, self.topk, dtype=torch.int32, device=dev)
        wg = torch.empty(self.world * cap, self.topk, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(xs, padded(x), group=self.group)
        dist.all_gather_into_tensor(idg, padded(ids, -1), group=self.group)
        dist.all_gather_into_tensor(wg, padded(weights), group=self.group)
        local = idg - self.rank * self.e_per
        local = torch.where((local >= 0) & (local < self.e_per), local, torch.full_like(local, -1))
        part = moe.experts_forward(xs, local.contiguous(), wg, ew).float()
        mine = torch.empty(cap, self.hidden_out, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(mine, part, group=self.group)
        out = mine[:t]
        if shared is not None:
            out = out + shared.float()
        return out.to(torch.bfloat16)


class HostExpertParallel:
    """The contract of `ExpertParallel.forward` on any device through a host all-gather (`allgather(obj) -> list`
    over the ranks: engine/dp.py has one over a torch.distributed group and one between threads). Every pair's
    expert output crosses as the bf16 row the owner computed and the caller sums its pairs in selection order, so
    the result is bitwise what one process holding every expert computes. For CPU runs of the data-parallel
    engine and as oracle."""

    def __init__(self, allgather, rank: int, world: int, experts: int):
        assert experts % world == 0
        self.allgather, self.rank, self.world = allgather, rank, world
        self.e_per = experts // world
        self.calls = 0

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: "moe.ExpertWeights", *,
                shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        dev = x.device
        self.calls += 1
        sent = self.allgather((x.cpu(), ids.cpu()))
        back = []
        for xs, sel in sent:                      # every rank's tokens through this rank's experts, pair by pair
            ys = torch.zeros(xs.shape[0], sel.shape[1], ew.fc2_rows, dtype=torch.bfloat16)
            if xs.shape[0]:
                one = torch.ones(xs.shape[0], 1, dtype=torch.float32, device=dev)
                for k in range(sel.shape[1]):
                    ys[:, k] = moe.experts_forward(xs.to(dev), sel[:, k:k + 1].contiguous().to(dev), one, ew,
                                                   id_base=self.rank * self.e_per).cpu()
            back.append(ys)
        got = self.allgather(back)
        mine = sum(got[r][self.rank].float() for r in range(self.world))      # exactly one owner per pair
        # selection-order fp32 sum, as the single-process combine does
        acc = torch.zeros(x.shape[0], ew.fc2_rows, dtype=torch.float32)
        for k in range(ids.shape[1]):
            acc += weights.float().cpu()[:, k:k + 1] * mine[:, k]
        if shared is not None:
            acc += shared.float().cpu()
        return acc.to(torch.bfloat16).to(dev)
