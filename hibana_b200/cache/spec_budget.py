"""What speculation will cost in memory, known before the cache pools are sized.

The memory plan (cache/ledger.py) hands everything left beside the weights to the KV and state pools, so what a
speculator allocates later must be set aside first: the verify scratch of recurrent models (snapshots of the
state after every verified position, or the compact inputs from which the accepted state is replayed), the drafter's
own weights where it has some, its KV (the MTP layer attends over one more KV layer: bytes per cached token, not a
fixed sum), the static buffers of the captured draft / verify graphs, and the dense draft laws of sampled block
drafts. `budget` returns (fixed bytes, extra bytes per KV slot). Pure arithmetic over the target's geometry.
Reference: hibana/cache/spec_budget.py:13-101.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..proposers.factory import MAX_DEPTHS
from ..target import GDN, MAMBA2, Target

MIB = 1 << 20


@dataclass(frozen=True)
class SpecConfig:
    name: str = "mtp"                     # mtp | ngram | dflash2
    depth: int = 3
    state_strategy: str = "reconstruct"   # snapshots | reconstruct
    draft_layers: int = 2                 # block drafter depth (dflash2)
    draft_width: int = 8                  # candidates per drafted position (dflash2)
    draft_window: int = 512               # positions of target features the block drafter attends over

    def __post_init__(self):
        if self.name not in MAX_DEPTHS or not 1 <= int(self.depth) <= MAX_DEPTHS[self.name]:
            raise ValueError(f"unsupported proposer / depth: {self.name} / {self.depth}")
        if self.state_strategy not in ("snapshots", "reconstruct"):
            raise ValueError(f"unsupported verify state strategy {self.state_strategy!r}")


def verify_bytes(batch: int, steps: int, strategy: str, t: Target) -> int:
    """Scratch the verify forward of `batch` requests x `steps` rows needs on a model with recurrent layers:
    "snapshots" keeps the full state after every row, "reconstruct" keeps the rows' compact inputs (conv inputs,
    decay and gate terms) and replays the accepted prefix into the pool."""
    total = 0
    for mixer, _ in t.layers:
        if mixer == MAMBA2:
            state = t.mamba_heads * t.mamba_head_dim * t.mamba_state * 4
            conv = t.mamba_conv_dim * (t.conv_width - 1) * 2
            compact = t.mamba_conv_dim * 2 + t.mamba_heads * 2 * 4          # x | B | C row, dt and exp(dt A)
        elif mixer == GDN:
            state = t.gdn_v_heads * t.gdn_head_dim * t.gdn_head_dim * 4
            conv = t.gdn_conv_dim * (t.conv_width - 1) * 2
            compact = t.gdn_conv_dim * 2 + t.gdn_v_heads * 2 * 4            # q | k | v row, decay and beta
        else:
            continue
        if strategy == "snapshots":
            total += batch * steps * (state + conv)
        else:
            total += batch * (state + conv) + batch * steps * compact        # one scratch slot + the rows' inputs
    return total


def budget(spec: Optional[SpecConfig], batch: int, t: Target, *, buckets: int = 3) -> tuple[int, int]:
    """(fixed bytes to set aside, extra bytes per KV slot) for serving `batch` requests with `spec`."""
    if spec is None:
        return 0, 0
    k1 = spec.depth + 1
    fixed = verify_bytes(batch, k1, spec.state_strategy, t)
    # static buffers of the captured rounds: hidden rows of every verified position, META, ids / slots / rows
    fixed += buckets * batch * k1 * (t.hidden * 2 * 3 + 64) + 4 * MIB
    # full-vocabulary logits of every verified row (relaxed / sampled acceptance reads them), fp32
    fixed += batch * k1 * (t.vocab // max(t.tp_size, 1)) * 4
    per_slot = 0
    if spec.name == "mtp":
        if not t.mtp_layers:
            raise ValueError(f"{t.name} has no MTP head to draft with")
        h = t.hidden
        ffn = t.ffn or max(t.expert_ffn * max(t.top_k, 1) // 2, 128)
        weights = 2 * h * h * 2 + (t.q_heads + 2 * t.kv_heads) * t.head_dim * h * 2 + t.q_heads * t.head_dim * h * 2 \
            + 3 * h * ffn * 2
        fixed += weights + 64 * MIB                                          # + allocator slack while loading
        esz = {"bf16": 2, "fp8": 1, "nvfp4": 0.5625}.get(t.kv_dtype, 2)
        per_slot = int(t.mtp_layers * 2 * max(t.kv_heads, 1) * t.head_dim * esz)
    elif spec.name == "dflash2":
        h = t.hidden
        fixed += spec.draft_layers * (4 * h * h + 3 * h * 2 * h) * 2         # the block drafter's own layers
        fixed += batch * spec.draft_window * spec.draft_layers * 2 * h * 2   # ring of target features per request
        fixed += batch * spec.depth * t.vocab * 4                            # dense draft laws of sampled requests
    return int(fixed), per_slot
