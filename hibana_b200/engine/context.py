"""Per-forward context handed from the executor to the model.

Holds positions, the KV slots of the new tokens, the block table of every sequence, recurrent-state slots and
which rows need logits. Every tensor is device-resident and, for graph replays, lives at a fixed address.
Reference: hibana/engine/context.py:23-93.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

PREFILL, DECODE, VERIFY = "prefill", "decode", "verify"


@dataclass
class ForwardContext:
    mode: str
    positions: torch.Tensor                    # int32 [T]
    slots: torch.Tensor                        # int32 [T] KV slot of each new token (0 = discard)
    kv_indices: torch.Tensor                   # int32 [B, max_ctx] slot of every position of every sequence
    ctx_len: torch.Tensor                      # int32 [B] context length including the new tokens
    q_indptr: Optional[torch.Tensor] = None    # int32 [B + 1]; None = exactly one row per sequence
    seq_rows: Optional[torch.Tensor] = None    # int32 [B] row of each sequence in kv_indices (None = identity)
    max_rows: int = 1                          # host bound on rows per sequence
    batch: int = 1
    state_slots: Optional[torch.Tensor] = None  # int32 [B] recurrent-state slot per sequence
    sample_rows: Optional[torch.Tensor] = None  # int64 [B'] rows whose logits are wanted (None = all rows)
    attn_splits: int = 1
    attn_workspace: Any = None
    max_ctx_host: int = 0
    # prefill chunk bookkeeping for recurrent layers
    seq_starts_host: Optional[list] = None      # rows per sequence on the host (prefill)
    has_initial_state: Optional[torch.Tensor] = None  # bool/int32 [B]: continue from the slot's state
    checkpoints: Optional[list] = None          # per sequence: list of (row offset, state slot) snapshots to emit
    extras: dict = field(default_factory=dict)
    comm: Any = None                            # tensor-parallel communicator (None = single GPU)
