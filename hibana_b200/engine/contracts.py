"""Typed boundaries between the engine and its pluggable parts (proposers, vision encoders).

A proposer drafts tokens; it never allocates target KV slots and never commits target state. Life cycle per request:
`ingest_prefill` (sees every target prefill chunk's hidden states) -> `start` -> per round `ready` / `propose`
-> `accepted_batch` once, after ALL target rows of the round are committed -> `release`. What a proposer can do is
declared in `Capabilities`; the engine checks them against what the configuration asks for (`check_capabilities`).
Reference: hibana/engine/contracts.py:36-125, docs/interfaces.md:140-161.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Protocol, Sequence, runtime_checkable

import torch


@dataclass(frozen=True)
class Capabilities:
    device_feedback: bool = False     # accepted tokens can be fed back without leaving the device
    checkpoint_cache: bool = False    # drafter state can be snapshotted with prefix-cache checkpoints
    stored_payload: bool = False      # drafter state can be serialised into the SSD tier's tail objects
    draft_head: bool = False          # owns a (possibly reduced) output head
    short_drafts: bool = False        # may return fewer than the requested number of tokens
    scored_drafts: bool = False       # returns an acceptance estimate per drafted token
    max_depth: int = 8


@dataclass
class Proposal:
    tokens: torch.Tensor                          # int64 [B, k]
    laws: Optional[torch.Tensor] = None           # fp32 [B, k, V] draft distributions (sampled acceptance)
    scores: Optional[torch.Tensor] = None         # fp32 [B, k] estimated acceptance per position
    lengths: Optional[Sequence[int]] = None       # valid drafts per request (short_drafts)


@dataclass
class VerifiedFeatures:
    hidden: torch.Tensor                          # target hidden states of the verified rows [rows, H]
    counts: Sequence[int]                         # emitted tokens per request; feature index count - 1 is current
    rows_per_request: int = 0


@runtime_checkable
class Proposer(Protocol):
    capabilities: Capabilities

    def ingest_prefill(self, req, hidden: torch.Tensor, start: int, count: int) -> None: ...
    def start(self, req) -> None: ...
    def ready(self, reqs: Sequence) -> bool: ...
    def propose(self, reqs: Sequence, depth: int) -> Proposal | torch.Tensor: ...
    def accepted_batch(self, reqs: Sequence, emitted: Sequence[Sequence[int]], features: Optional[VerifiedFeatures]) -> None: ...
    def release(self, req) -> None: ...


@dataclass
class ProposerRequirements:
    sampled: bool = False             # needs draft laws
    row_budget: bool = False          # needs scored drafts
    depth: int = 1
    ssd_payload: bool = False


def check_capabilities(caps: Capabilities, need: ProposerRequirements) -> None:
    problems = []
    if need.depth > caps.max_depth:
        problems.append(f"depth {need.depth} exceeds the proposer's maximum {caps.max_depth}")
    if need.row_budget and not caps.scored_drafts:
        problems.append("row budgeting needs scored drafts")
    if need.ssd_payload and not caps.stored_payload:
        problems.append("the SSD tier is asked to store drafter state the proposer cannot serialise")
    if problems:
        raise ValueError("; ".join(problems))


@runtime_checkable
class VisionEncoder(Protocol):
    def encode(self, pixels: torch.Tensor) -> torch.Tensor: ...
    tokens_per_image: int
