"""Requests and per-request sampling parameters.

A request owns its prompt, emitted tokens, sampling law and timing marks; physical resources (KV slots, state
slot, radix lock) hang off its `RequestState` base and are only moved by the StateManager.
Reference: hibana/engine/request.py:15-108, hibana/engine/sampler.py:21-84.
"""
from __future__ import annotations

import enum
import itertools
import time
from dataclasses import dataclass, field
from typing import Any, Optional

MAX_STOPS = 8


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    max_tokens: int = 128
    stop_ids: tuple = ()
    ignore_eos: bool = False
    seed: Optional[int] = None
    accept_top_k: int = 1            # relaxed speculative acceptance: drafted token within target top-K ...
    accept_margin: float = 0.0       # ... and within this many logits of the argmax
    accept_soft: float = 0.0         # sampled acceptance slack s: accept when u*q < e^s * p
    logprobs: int = 0
    constraint: Any = None           # engine.grammar.Constraint: the output must match this grammar

    def __post_init__(self) -> None:
        if self.temperature < 0 or self.top_p <= 0 or self.top_p > 1 or self.top_k < 0:
            raise ValueError("invalid sampling parameters")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        if len(self.stop_ids) > 64:
            raise ValueError("too many stop ids")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


class State(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    RUNNING = "running"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"


_ids = itertools.count(1)


@dataclass
class RequestState:
    """Physical state of a request; fields are written by the StateManager only."""
    kv_slots: list = field(default_factory=list)     # slot of every committed + pending position
    state_slot: int = 0                              # recurrent-state slot (0 = none)
    table_row: int = -1                              # row in the device block table
    committed_len: int = 0                           # tokens whose KV / state are final
    cached_len: int = 0                              # prefix length served from the radix cache at admission
    shared_len: int = 0                              # kv_slots[:shared_len] belong to the radix tree
    branch_at: int = 0                               # where the prompt left an existing cached path
    lock: Any = None                                 # radix TreeLock
    cacheable: bool = True
    reserved: int = 0                                # slots reserved for the step in flight


@dataclass
class Request(RequestState):
    prompt_ids: list = field(default_factory=list)
    params: SamplingParams = field(default_factory=SamplingParams)
    rid: int = field(default_factory=lambda: next(_ids))
    output_ids: list = field(default_factory=list)
    state: State = State.WAITING
    prefilled: int = 0                               # prompt tokens already run through the model
    finish_reason: Optional[str] = None
    eos_id: Optional[int] = None
    media: Any = None
    grammar: Any = None                              # engine.grammar.GrammarState of a constrained request
    arrival: float = field(default_factory=time.monotonic)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    waits: int = 0
    draws: int = 0                                   # RNG offset: number of sampling draws consumed
    stream_cursor: int = 0
    rounds: list = field(default_factory=list)       # per speculative round accepted counts (traces)
    token_logprobs: list = field(default_factory=list)   # per emitted token (logprob, [(token, logprob)]) when asked for

    @property
    def all_ids(self) -> list:
        return self.prompt_ids + self.output_ids

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def remaining(self) -> int:
        return self.params.max_tokens - len(self.output_ids)

    @property
    def done(self) -> bool:
        return self.state in (State.FINISHED, State.CANCELLED, State.FAILED)

    @property
    def seed(self) -> int:
        return self.params.seed if self.params.seed is not None else self.rid * 0x9E3779B1

    def push(self, token: int) -> bool:
        """Appends an emitted token; returns True when the request finished with it."""
        if self.done:
            return True
        if self.first_token_time is None:
            self.first_token_time = time.monotonic()
        self.output_ids.append(int(token))
        if self.grammar is not None:
            self.grammar.push(int(token))
        stop = int(token) in self.params.stop_ids or (
            self.eos_id is not None and not self.params.ignore_eos and int(token) == self.eos_id)
        if stop:
            self._finish("stop")
        elif len(self.output_ids) >= self.params.max_tokens:
            self._finish("length")
        return self.done

    def _finish(self, reason: str) -> None:
        self.state = State.FINISHED
        self.finish_reason = reason
        self.finish_time = time.monotonic()

    def cancel(self) -> None:
        if not self.done:
            self.state = State.CANCELLED
            self.finish_reason = "cancelled"
            self.finish_time = time.monotonic()

    def fail(self, reason: str = "error") -> None:
        if not self.done:
            self.state = State.FAILED
            self.finish_reason = reason
            self.finish_time = time.monotonic()

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival
