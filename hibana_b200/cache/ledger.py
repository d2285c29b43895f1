"""Memory plan: how many KV slots and recurrent-state slots fit beside the weights.

    free after weights - first-use reserve (CUDA context, library workspaces, allocator slack)
                       - activations of the largest forward (prefill chunk)
                       - CUDA graphs (per captured bucket)
                       - fixed workspaces (attention split partials, communicator heaps)
    = pool budget; pools cost `POOL_COST` x their payload (allocator rounding, block tables).
State slots come first (floor 2 x max_batch + 1 (+1 with an SSD restore in flight): a request pins at most its own
slot and one checkpoint between steps), then the rest goes to KV slots; `fraction` leaves headroom. The plan is pure
arithmetic over numbers the caller measures (free bytes, weight bytes), so it is testable without a GPU.
Reference: hibana/cache/ledger.py:119-196 (constants POOL_COST 1.04, first use 2.25 GiB, activations 1 GiB),
docs/memory_plan.md.
"""
from __future__ import annotations

from dataclasses import dataclass, field

GIB = 1 << 30
POOL_COST = 1.04
FIRST_USE_BYTES = int(2.25 * GIB)
ACTIVATION_BYTES = 1 * GIB


@dataclass
class Plan:
    kv_slots: int
    state_slots: int
    kv_bytes: int
    state_bytes: int
    graph_bytes: int
    workspace_bytes: int
    reserve_bytes: int
    notes: list = field(default_factory=list)

    def as_dict(self) -> dict:
        return {k: getattr(self, k) for k in ("kv_slots", "state_slots", "kv_bytes", "state_bytes", "graph_bytes",
                                              "workspace_bytes", "reserve_bytes", "notes")}


def graph_bytes(buckets, hidden: int, vocab: int, layers: int) -> int:
    """Private pool of one captured decode graph per bucket: a few activation rows per layer boundary + logits."""
    return sum(b * (hidden * 2 * 12 + vocab * 4) + (2 << 20) for b in buckets) + layers * (64 << 10)


def activation_bytes(chunk_tokens: int, hidden: int, ffn: int, q_dim: int, vocab_rows: int, vocab: int) -> int:
    """Peak transient memory of one prefill forward (one layer live at a time)."""
    per_token = 2 * (3 * hidden + 2 * q_dim + 3 * ffn) + ffn       # bf16 activations + packed FP4 copies
    return max(chunk_tokens * per_token + vocab_rows * vocab * 4, 64 << 20)


class Ledger:
    def __init__(self, free_bytes: int, *, fraction: float = 0.92):
        self.free, self.fraction = int(free_bytes), fraction

    def plan(self, *, kv_bytes_per_token: int, state_bytes_per_slot: int = 0, max_batch: int = 64,
             max_ctx: int = 4096, graph: int = 0, workspace: int = 0, activations: int = ACTIVATION_BYTES,
             first_use: int = FIRST_USE_BYTES, want_state_slots: int = 0, ssd_restore: bool = False,
             min_kv_slots: int = 0) -> Plan:
        notes = []
        budget = int(self.free * self.fraction) - first_use - activations - graph - workspace
        reserve = self.free - max(budget, 0)
        if budget <= 0:
            raise MemoryError(f"nothing left for the pools: {self.free / GIB:.1f} GiB free, "
                              f"{(first_use + activations + graph + workspace) / GIB:.1f} GiB of fixed needs")
        state_slots = state_bytes = 0
        if state_bytes_per_slot:
            floor = 2 * max_batch + 1 + (1 if ssd_restore else 0)
            state_slots = max(floor, want_state_slots)
            state_bytes = int(state_slots * state_bytes_per_slot * POOL_COST)
            if state_bytes > budget // 2:
                state_slots = max(floor, int(budget // 2 / (state_bytes_per_slot * POOL_COST)))
                state_bytes = int(state_slots * state_bytes_per_slot * POOL_COST)
                notes.append(f"state slots cut to {state_slots} (half of the pool budget)")
            if state_slots < floor or state_bytes > budget:
                raise MemoryError(f"the floor of {floor} state slots does not fit")
        kv_budget = budget - state_bytes
        kv_slots = int(kv_budget / (kv_bytes_per_token * POOL_COST)) if kv_bytes_per_token else 0
        floor_kv = max(min_kv_slots, max_ctx + 64)
        if kv_bytes_per_token and kv_slots < floor_kv:
            raise MemoryError(f"KV pool of {kv_slots} slots cannot hold one request of {max_ctx} tokens")
        useful = max_batch * max_ctx * 4
        if kv_slots > useful:
            notes.append(f"KV pool capped at 4 x max_batch x max_ctx = {useful} slots")
            kv_slots = useful
        return Plan(kv_slots, state_slots, int(kv_slots * kv_bytes_per_token * POOL_COST), state_bytes, graph, workspace,
                    reserve, notes)

    def above_floor(self, plan: Plan, max_batch: int) -> bool:
        return plan.state_slots == 0 or plan.state_slots > 2 * max_batch + 1
