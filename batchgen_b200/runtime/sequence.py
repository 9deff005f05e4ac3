"""Sequence state machine and the page arithmetic attached to it.

States and edges follow batchgen/sequence.py:58-66,134-142:

    QUEUEING -> IN_PREFILL -> PREFILLED -> IN_DECODE <-> ON_HOLD -> COMPLETED
                                  ^                         |
    EVICTED (KV dropped, token ids kept) ---recompute-------+

``PREFILLED`` means the KV exists but is not in the decode batch; ``ON_HOLD`` means the row left the
decode batch (its KV lives in the host tier or stays parked on the GPU); ``EVICTED`` keeps only token
ids and re-enters through prefill.  Page formulas are the ones of batchgen/sequence.py:464-625.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional


class SequenceStatus(enum.IntEnum):
    QUEUEING = 0
    IN_PREFILL = 1
    PREFILLED = 2
    IN_DECODE = 3
    ON_HOLD = 4
    COMPLETED = 5
    EVICTED = 6


S = SequenceStatus
VALID_TRANSITIONS: Dict[SequenceStatus, frozenset] = {
    S.QUEUEING: frozenset({S.IN_PREFILL, S.COMPLETED}),
    S.IN_PREFILL: frozenset({S.PREFILLED, S.COMPLETED, S.QUEUEING}),
    S.PREFILLED: frozenset({S.IN_DECODE, S.ON_HOLD, S.EVICTED, S.COMPLETED}),
    S.IN_DECODE: frozenset({S.ON_HOLD, S.COMPLETED, S.EVICTED}),
    S.ON_HOLD: frozenset({S.IN_DECODE, S.EVICTED, S.COMPLETED}),
    S.EVICTED: frozenset({S.IN_PREFILL, S.COMPLETED}),
    S.COMPLETED: frozenset(),
}

# named edges (batchgen/sequence.py:680-692)
EDGE_NAMES = {
    (S.QUEUEING, S.IN_PREFILL): "PREFILL", (S.EVICTED, S.IN_PREFILL): "PREFILL",
    (S.IN_PREFILL, S.PREFILLED): "PREFILL", (S.PREFILLED, S.IN_DECODE): "DECODE_ENTRY",
    (S.ON_HOLD, S.IN_DECODE): "DECODE_ENTRY", (S.IN_DECODE, S.ON_HOLD): "CAPACITY_HOLD",
    (S.PREFILLED, S.ON_HOLD): "CAPACITY_HOLD", (S.IN_DECODE, S.EVICTED): "BOUNDARY",
    (S.ON_HOLD, S.EVICTED): "BOUNDARY", (S.PREFILLED, S.EVICTED): "BOUNDARY",
}


class InvalidTransition(RuntimeError):
    pass


class Priority(enum.IntEnum):
    NORMAL = 0
    HIGH = 1


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    max_new_tokens: int = 16
    ignore_eos: bool = False
    seed: Optional[int] = None


@dataclass
class PageBufferConfig:
    """Runtime-overridable buffer sizes (batchgen/sequence.py:29-54)."""
    page_size: int = 64
    initial_gpu_page_buffer: int = 32
    extension_gpu_page_buffer: int = 4
    decision_frequency_pages: int = 2

    @property
    def decision_interval(self) -> int:
        return self.decision_frequency_pages * self.page_size


@dataclass
class Sequence:
    global_idx: int
    prompt_ids: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    custom_id: str = ""
    batch_id: str = ""
    priority: Priority = Priority.NORMAL
    status: SequenceStatus = SequenceStatus.QUEUEING
    output_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    assigned_rank: int = 0
    decode_dp_group: int = 0
    prefill_order: Optional[int] = None
    # KV bookkeeping
    gpu_pages: List[int] = field(default_factory=list)      # physical GPU pages in order
    host_pages: List[int] = field(default_factory=list)     # physical host pages in order
    state_slot: int = -1                                    # recurrent-state slot (models with KDA layers)
    state_item: int = -1                                    # host item holding the state while the row is on hold
    session_id: Optional[str] = None                        # agent session this request is a turn of
    inflight_tokens: int = 0                                # decode steps launched whose token is not on the host yet
    decode_owner: int = -1                                  # TP rank whose KV copy is kept current (request-split decode)
    num_cached_tokens: int = 0                              # tokens whose KV exists (either tier)
    cached_prefix_tokens: int = 0                           # tokens served by the prefix cache
    had_initial_gpu_reservation: bool = False
    host_token_capacity: int = 0
    # eviction bookkeeping
    total_decoded_before_eviction: int = 0
    reentry_decoded_baseline: int = 0
    history: List[str] = field(default_factory=list)

    # ------------------------------------------------------------------ state machine
    def transition(self, new: SequenceStatus) -> None:
        if new not in VALID_TRANSITIONS[self.status]:
            raise InvalidTransition(f"seq {self.global_idx}: {self.status.name} -> {new.name}")
        self.history.append(f"{self.status.name}->{new.name}")
        self.status = new

    # ------------------------------------------------------------------ token views
    @property
    def all_ids(self) -> List[int]:
        return self.prompt_ids + self.output_ids

    @property
    def context_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def num_decoded(self) -> int:
        return len(self.output_ids)

    def is_finished(self, eos_token_id: int) -> Optional[str]:
        if self.num_decoded >= self.params.max_new_tokens:
            return "length"
        if self.output_ids and not self.params.ignore_eos and self.output_ids[-1] == eos_token_id:
            return "stop"
        return None

    def evict(self) -> None:
        """Drop all KV; keep token ids so the row can be recomputed through prefill."""
        self.total_decoded_before_eviction = self.num_decoded
        self.reentry_decoded_baseline = self.num_decoded
        self.gpu_pages, self.host_pages = [], []
        self.num_cached_tokens = 0
        self.had_initial_gpu_reservation = False
        self.host_token_capacity = 0
        self.decode_owner = -1                # prefill rebuilds the KV on every rank: any owner will do afterwards
        self.transition(S.EVICTED)


# ---------------------------------------------------------------------- page arithmetic
def pages_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


def gpu_pages_first_load(ctx: int, buf: PageBufferConfig, kv_token_budget: int) -> int:
    """ceil(min(ctx + initial_buffer * page, budget) / page)."""
    return pages_for(min(ctx + buf.initial_gpu_page_buffer * buf.page_size, kv_token_budget), buf.page_size)


def gpu_pages_in_decode(ctx: int, had_initial: bool, buf: PageBufferConfig, kv_token_budget: int) -> int:
    b = buf.extension_gpu_page_buffer if had_initial else buf.initial_gpu_page_buffer
    return pages_for(min(ctx + b * buf.page_size, kv_token_budget), buf.page_size)


def extra_gpu_pages_needed(ctx: int, allocated: int, buf: PageBufferConfig, kv_token_budget: int) -> int:
    want = pages_for(min(ctx + buf.extension_gpu_page_buffer * buf.page_size, kv_token_budget), buf.page_size)
    return max(0, want - allocated)


def host_growth_due(ctx: int, host_token_capacity: int, buf: PageBufferConfig) -> bool:
    return host_token_capacity - ctx <= buf.extension_gpu_page_buffer * buf.page_size


def host_pages_at_admission(prompt_len: int, chunk: int, buf: PageBufferConfig, kv_token_budget: int,
                            replication: int = 1) -> int:
    a = prompt_len + chunk
    b = (pages_for(prompt_len + 1, buf.page_size) + buf.initial_gpu_page_buffer) * buf.page_size
    return pages_for(min(max(a, b), kv_token_budget), buf.page_size) * replication


class AdaptiveChunkSizer:
    """EMA of decoded lengths -> host growth chunk (batchgen/continuous_batching.py:430-481)."""

    def __init__(self, initial: int, lo: int = 256, hi: int = 65536, alpha: float = 0.2, warmup: int = 10):
        self.chunk, self.lo, self.hi, self.alpha, self.warmup = initial, lo, hi, alpha, warmup
        self.ema: Optional[float] = None
        self.n = 0

    def observe(self, decoded_len: int) -> int:
        self.n += 1
        self.ema = decoded_len if self.ema is None else (1 - self.alpha) * self.ema + self.alpha * decoded_len
        if self.n >= self.warmup:
            c = min(max(self.ema * 1.5, self.lo), self.hi)
            self.chunk = int(math.ceil(c / 64.0)) * 64
        return self.chunk
