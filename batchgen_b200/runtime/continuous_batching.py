"""Continuous-batching policy: adaptive host-KV chunk size, growth-driven eviction planning, and the choice
of held sequences to bring back onto the GPU.  All functions are pure and deterministic (stable tie-breaks on
``global_idx`` then uuid), because every rank evaluates them on the same snapshot and must agree.

Reference parity: batchgen/continuous_batching.py:430 (AdaptiveChunkSizer), :484
(select_sequences_for_eviction), :553-575 (growth cost-aware key), :578-700
(plan_host_kv_growth_evictions), :708-830 (select_sequences_for_loading).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from fractions import Fraction
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

PAGE_TOKENS = 64


class EvictionStrategy(enum.Enum):
    SHORTEST_FIRST = "shortest_first"        # evict the rows that decoded least (cheapest to redo)
    LONGEST_FIRST = "longest_first"
    FIFO = "fifo"
    GROWTH_COST_AWARE = "growth_cost_aware"  # most deficit pages closed per token a re-prefill recomputes


class LoadingStrategy(enum.Enum):
    LONGEST_FIRST = "longest_first"
    SHORTEST_FIRST = "shortest_first"
    FIFO = "fifo"


class AdaptiveChunkSizer:
    """Host-KV reservation chunk that follows an exponential moving average of completed decode lengths:
    chunk = clamp(multiplier * ema), rounded up to a page, once 10 completions have been seen."""

    def __init__(self, initial_chunk: int = 8192, min_chunk: int = 1024, max_chunk: int = 65536,
                 ema_alpha: float = 0.1, multiplier: float = 1.5, warmup: int = 10):
        self.current_chunk, self.min_chunk, self.max_chunk = initial_chunk, min_chunk, max_chunk
        self.ema_alpha, self.multiplier, self.warmup = ema_alpha, multiplier, warmup
        self.ema_decode_length: Optional[float] = None
        self.completed_count = 0

    def report_completion(self, decoded_length: int) -> None:
        if self.ema_decode_length is None:
            self.ema_decode_length = float(decoded_length)
        else:
            self.ema_decode_length += self.ema_alpha * (decoded_length - self.ema_decode_length)
        self.completed_count += 1
        if self.completed_count >= self.warmup:
            target = min(self.max_chunk, max(self.min_chunk, self.ema_decode_length * self.multiplier))
            self.current_chunk = math.ceil(int(target) / PAGE_TOKENS) * PAGE_TOKENS

    def get_chunk_size(self) -> int:
        return self.current_chunk


def _order(cands: Iterable[Tuple[str, Dict[str, Any]]], strategy: EvictionStrategy, page_key: str):
    def gidx(st):
        return st.get("global_idx", float("inf"))
    if strategy is EvictionStrategy.GROWTH_COST_AWARE:
        def key(item):
            uuid, st = item
            for k in ("growth_pages", "recompute_tokens"):
                if k not in st:
                    raise ValueError(f"GROWTH_COST_AWARE eviction candidate {uuid} has no {k!r}")
            benefit = int(st.get(page_key, 0) or 0) + int(st["growth_pages"])
            return (st.get("priority", 0), Fraction(-benefit, max(1, int(st["recompute_tokens"]))), gidx(st), uuid)
    elif strategy is EvictionStrategy.SHORTEST_FIRST:
        def key(item):
            return (item[1].get("priority", 0), item[1].get("decoded_length", 0), gidx(item[1]), item[0])
    elif strategy is EvictionStrategy.LONGEST_FIRST:
        def key(item):
            return (item[1].get("priority", 0), -item[1].get("decoded_length", 0), gidx(item[1]), item[0])
    else:
        def key(item):
            return (item[1].get("priority", 0), gidx(item[1]), item[0])
    return sorted(cands, key=key)


def select_sequences_for_eviction(sequences: Sequence[Tuple[str, Dict[str, Any]]], pages_to_free: int,
                                  strategy: EvictionStrategy = EvictionStrategy.SHORTEST_FIRST,
                                  page_key: str = "gpu_pages_allocated") -> Tuple[List[str], int]:
    """Victims (normal priority before high) until at least ``pages_to_free`` pages come back."""
    if strategy is EvictionStrategy.GROWTH_COST_AWARE:
        raise ValueError("GROWTH_COST_AWARE scores host-KV growth debt: use plan_host_kv_growth_evictions")
    out, freed = [], 0
    if pages_to_free <= 0:
        return out, freed
    for uuid, st in _order(sequences, strategy, page_key):
        if freed >= pages_to_free:
            break
        pages = int(st.get(page_key, 0) or 0)
        if pages > 0:
            out.append(uuid)
            freed += pages
    return out, freed


@dataclass
class HostKVGrowthEvictionPlan:
    evicted_uuids: List[str] = field(default_factory=list)
    freed_pages: int = 0
    remaining_growth_uuids: List[str] = field(default_factory=list)
    remaining_growth_pages: List[int] = field(default_factory=list)
    remaining_growth_needed: int = 0
    expected_free_pages: int = 0
    required_free_pages: int = 0
    growth_feasible_after_eviction: bool = True


def plan_host_kv_growth_evictions(*, active_uuids: Sequence[str], completed_uuids: Sequence[str],
                                  host_growth_uuids: Sequence[str], host_growth_pages: Sequence[int],
                                  eviction_candidates: Sequence[Tuple[str, Dict[str, Any]]], free_pages: int,
                                  total_pages: int, completed_pages: int, reclaimable_pages: int = 0,
                                  strategy: EvictionStrategy = EvictionStrategy.SHORTEST_FIRST,
                                  page_key: str = "host_owned_pages") -> HostKVGrowthEvictionPlan:
    """After a page boundary every row that stays active must be able to grow.  The growth debt is covered,
    in order, by free pages, pages released by completed rows, reclaimable prefix-cache pages and finally
    the owned pages of evicted rows (which also retire their own debt).  Eviction is strictly growth driven:
    a full pool with no debt evicts nobody."""
    if len(host_growth_uuids) != len(host_growth_pages):
        raise ValueError("host_growth_uuids and host_growth_pages must align")
    done, active = set(completed_uuids), set(active_uuids)
    total = max(total_pages, 0)
    base_free = min(total, max(free_pages, 0) + max(completed_pages, 0) + max(reclaimable_pages, 0))
    debt = {u: p for u, p in zip(host_growth_uuids, host_growth_pages) if p > 0 and u in active and u not in done}
    need = sum(debt.values())
    plan = HostKVGrowthEvictionPlan()
    for uuid, st in _order(eviction_candidates, strategy, page_key):
        if min(total, base_free + plan.freed_pages) >= need:
            break
        pages = int(st.get(page_key, 0) or 0)
        if uuid in done or pages <= 0:
            continue
        plan.evicted_uuids.append(uuid)
        plan.freed_pages += pages
        need -= debt.pop(uuid, 0)
    plan.remaining_growth_uuids = [u for u in host_growth_uuids if u in debt]
    plan.remaining_growth_pages = [debt[u] for u in plan.remaining_growth_uuids]
    plan.remaining_growth_needed = need
    plan.expected_free_pages = min(total, base_free + plan.freed_pages)
    plan.required_free_pages = max(need, 0)
    plan.growth_feasible_after_eviction = need == 0 or plan.expected_free_pages >= need
    return plan


def select_sequences_for_loading(candidates: Dict[str, Dict[str, Any]], per_rank_free_pages: Sequence[int],
                                 exclude_uuids: Set[str], strategy: LoadingStrategy = LoadingStrategy.LONGEST_FIRST,
                                 get_global_idx_fn: Optional[Callable[[str], int]] = None, group_size: int = 1,
                                 per_group_seq_slots: Optional[Sequence[int]] = None
                                 ) -> Tuple[List[str], Dict[int, int]]:
    """Held sequences to load back, charged to their capacity bucket: a rank (pure DP) or a decode group of
    ``group_size`` ranks whose capacity is its tightest rank.  Returns (uuids, pages used per bucket)."""
    if group_size <= 0 or len(per_rank_free_pages) % group_size:
        raise ValueError(f"group_size={group_size} must divide the number of ranks={len(per_rank_free_pages)}")
    n_groups = len(per_rank_free_pages) // group_size
    cap = [min(per_rank_free_pages[g * group_size:(g + 1) * group_size]) for g in range(n_groups)]
    used = {g: 0 for g in range(n_groups)}
    loaded = [0] * n_groups

    def key(item):
        uuid, info = item
        gi = get_global_idx_fn(uuid) if get_global_idx_fn else float("inf")
        n = info.get("decoded_length", 0)
        if strategy is LoadingStrategy.LONGEST_FIRST:
            return (-n, gi, uuid)
        if strategy is LoadingStrategy.SHORTEST_FIRST:
            return (n, gi, uuid)
        return (gi, uuid)

    out: List[str] = []
    for uuid, info in sorted(((u, i) for u, i in candidates.items() if u not in exclude_uuids), key=key):
        g = info.get("decode_dp_group") if group_size > 1 else info.get("assigned_rank", 0)
        if not isinstance(g, int) or not 0 <= g < n_groups:
            raise ValueError(f"candidate {uuid} has no valid capacity bucket for group_size={group_size}")
        pages = int(info.get("pages_needed", 0))
        if pages <= 0:
            continue
        if per_group_seq_slots is not None and loaded[g] >= per_group_seq_slots[g]:
            continue
        if used[g] + pages <= cap[g]:
            used[g] += pages
            loaded[g] += 1
            out.append(uuid)
    return out, used
