"""Pure scheduling policy: every function here is a deterministic function of a snapshot, so all
ranks compute the same answer from the same gathered state without another collective, and the
whole policy layer is unit-testable on CPU.

Covers (with the reference location of the behaviour being reproduced):
  * prepack_ffd               first-fit-decreasing packing into token-capped micro-batches
                              (batchgen/prefill/prepack.py:55-365)
  * assign_ranks_l2           FFD on sum of prompt_length^2 (batchgen/batchgen_worker.py:1987-2033)
  * select_prefill_batch      EVICTED first, skip-and-continue page budget walk with a marginal
                              shared-prefix charge (batchgen/worker/prefill.py:297-441)
  * select_decode_batch       PREFILLED + ON_HOLD in global order under page and row budgets
                              (batchgen/worker/decode.py:201-320)
  * compute_boundary_decisions completions, growth-driven eviction, extension or ON_HOLD, loading
                              (batchgen/worker/boundary.py:95-564; continuous_batching.py:553-823)
  * plan_kv_migration         host-KV balancing between nodes (batchgen/worker/kv_manager.py:676-800)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from fractions import Fraction
from typing import Dict, Iterable, List, Optional, Sequence as Seq, Tuple

from .sequence import (PageBufferConfig, Priority, Sequence, SequenceStatus, extra_gpu_pages_needed,
                       gpu_pages_first_load, pages_for)

S = SequenceStatus


# ---------------------------------------------------------------------- prepack
@dataclass
class MicroBatch:
    seq_indices: List[int]
    lengths: List[int]

    @property
    def tokens(self) -> int:
        return sum(self.lengths)

    @property
    def cu_seqlens(self) -> List[int]:
        out = [0]
        for n in self.lengths:
            out.append(out[-1] + n)
        return out


def prepack_ffd(lengths: Seq[int], token_cap: int, l2_cap: Optional[int] = None) -> List[MicroBatch]:
    """Pack sequences (by index) into micro-batches of at most ``token_cap`` tokens, longest first,
    first fit.  A sequence longer than the cap gets a micro-batch of its own (single-long-sequence
    guard).  ``l2_cap`` additionally bounds sum(len^2) per micro-batch (attention cost)."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    bins: List[MicroBatch] = []
    loads: List[Tuple[int, int]] = []
    for i in order:
        n = lengths[i]
        if n <= 0:
            continue
        placed = False
        for b, (tok, l2) in enumerate(loads):
            if tok + n <= token_cap and (l2_cap is None or l2 + n * n <= l2_cap):
                bins[b].seq_indices.append(i)
                bins[b].lengths.append(n)
                loads[b] = (tok + n, l2 + n * n)
                placed = True
                break
        if not placed:
            bins.append(MicroBatch([i], [n]))
            loads.append((n, n * n))
    return bins


def assign_ranks_l2(prompt_lengths: Seq[int], num_ranks: int, initial_load: Optional[Seq[int]] = None) -> List[int]:
    """Longest first, each to the rank with the smallest running sum of length^2."""
    load = list(initial_load) if initial_load is not None else [0] * num_ranks
    out = [0] * len(prompt_lengths)
    for i in sorted(range(len(prompt_lengths)), key=lambda i: (-prompt_lengths[i], i)):
        r = min(range(num_ranks), key=lambda r: (load[r], r))
        out[i] = r
        load[r] += prompt_lengths[i] ** 2
    return out


# ---------------------------------------------------------------------- shared-prefix ledger
class SharedPrefixLedger:
    """Marginal page charging for sequences that share prefix segments: the first reader of a
    segment pays for it, later readers pay only their private tail (floor one page)."""

    def __init__(self):
        self._refs: Dict[object, int] = {}
        self._saved: Optional[Dict[object, int]] = None

    def preview(self, total_pages: int, segments: Seq[Tuple[object, int]]) -> int:
        shared = sum(p for key, p in segments if self._refs.get(key, 0) > 0)
        return max(1, total_pages - shared)

    def charge(self, total_pages: int, segments: Seq[Tuple[object, int]]) -> int:
        cost = self.preview(total_pages, segments)
        for key, _ in segments:
            self._refs[key] = self._refs.get(key, 0) + 1
        return cost

    def release(self, segments: Seq[Tuple[object, int]]) -> int:
        freed = 0
        for key, p in segments:
            self._refs[key] -= 1
            if self._refs[key] == 0:
                del self._refs[key]
                freed += p
        return freed

    def savepoint(self) -> None:
        self._saved = dict(self._refs)

    def rollback(self) -> None:
        assert self._saved is not None
        self._refs, self._saved = self._saved, None


# ---------------------------------------------------------------------- prefill admission
@dataclass
class PrefillSelection:
    admitted: List[int] = field(default_factory=list)          # global_idx in admission order
    pages_charged: Dict[int, int] = field(default_factory=dict)
    skipped: List[int] = field(default_factory=list)


def select_prefill_batch(seqs: Iterable[Sequence], free_pages: int, buf: PageBufferConfig,
                         reserve_decode_tokens: int = 0, max_sequences: Optional[int] = None,
                         prefix_segments: Optional[Dict[int, List[Tuple[object, int]]]] = None,
                         ledger: Optional[SharedPrefixLedger] = None,
                         reclaimable_pages: int = 0) -> PrefillSelection:
    """Walk candidates (EVICTED first by least wasted recompute, then QUEUEING by prefill order) and
    admit every one whose marginal page charge still fits; a candidate that does not fit is skipped
    and the walk continues."""
    ev = sorted((s for s in seqs if s.status == S.EVICTED),
                key=lambda s: (-s.total_decoded_before_eviction, s.global_idx))
    qu = sorted((s for s in seqs if s.status == S.QUEUEING),
                key=lambda s: (s.prefill_order if s.prefill_order is not None else s.global_idx, s.global_idx))
    budget = free_pages + reclaimable_pages
    ledger = ledger or SharedPrefixLedger()
    sel = PrefillSelection()
    for s in ev + qu:
        if max_sequences is not None and len(sel.admitted) >= max_sequences:
            break
        need_tokens = s.context_len + reserve_decode_tokens
        total = pages_for(need_tokens, buf.page_size)
        segs = (prefix_segments or {}).get(s.global_idx, [])
        cost = ledger.preview(total, segs)
        if cost <= budget:
            ledger.charge(total, segs)
            budget -= cost
            sel.admitted.append(s.global_idx)
            sel.pages_charged[s.global_idx] = cost
        else:
            sel.skipped.append(s.global_idx)
    return sel


class PrefillProgressGuard:
    """Turns an endless sequence of empty admissions into a named failure
    (batchgen/worker/prefill.py:598)."""

    def __init__(self, limit: int = 64):
        self.limit, self.count, self.last_state = limit, 0, None

    def observe(self, admitted: int, live: int, state_digest) -> None:
        if admitted > 0 or live > 0 or state_digest != self.last_state:
            self.count = 0
        else:
            self.count += 1
        self.last_state = state_digest
        if self.count >= self.limit:
            raise RuntimeError("[SCHED_INVARIANT] prefill admission made no progress "
                               f"for {self.limit} consecutive waves with nothing live")


# ---------------------------------------------------------------------- decode admission
class DecodeCapacityError(RuntimeError):
    pass


def select_decode_batch(seqs: Iterable[Sequence], free_pages: Dict[int, int], in_decode_rows: Dict[int, int],
                        max_rows_per_bucket: int, buf: PageBufferConfig, kv_token_budget: int,
                        total_pages_per_bucket: Optional[int] = None,
                        resident: Optional[set] = None) -> List[int]:
    """Admit PREFILLED + ON_HOLD rows in global order while their GPU page need fits the bucket's
    free pages and the bucket has row slots left.  ``resident`` holds rows whose KV already sits in
    the GPU pool (they need only the growth buffer).  Buckets are ranks (DP) or serve groups."""
    free = dict(free_pages)
    rows = dict(in_decode_rows)
    out: List[int] = []
    cands = sorted((s for s in seqs if s.status in (S.PREFILLED, S.ON_HOLD)), key=lambda s: s.global_idx)
    for s in cands:
        b = s.decode_dp_group
        need = gpu_pages_first_load(s.context_len, buf, kv_token_budget)
        if total_pages_per_bucket is not None and need > total_pages_per_bucket:
            raise DecodeCapacityError(f"seq {s.global_idx} needs {need} pages; a replica has {total_pages_per_bucket}")
        have = len(s.gpu_pages) if (resident and s.global_idx in resident) else 0
        marginal = max(0, need - have)
        if rows.get(b, 0) >= max_rows_per_bucket:
            continue
        if marginal <= free.get(b, 0):
            free[b] = free.get(b, 0) - marginal
            rows[b] = rows.get(b, 0) + 1
            out.append(s.global_idx)
    return out


# ---------------------------------------------------------------------- boundary decisions
@dataclass
class BoundaryDecisions:
    completed: List[int] = field(default_factory=list)
    evicted: List[int] = field(default_factory=list)
    extend: Dict[int, int] = field(default_factory=dict)      # global_idx -> extra GPU pages
    on_hold: List[int] = field(default_factory=list)
    load: List[int] = field(default_factory=list)
    host_growth: Dict[int, int] = field(default_factory=dict)  # global_idx -> extra host pages
    scheduler_error: Optional[str] = None


def _victim_key(s: Sequence, deficit_pages: int):
    """Most deficit closed per recompute token first (GROWTH_COST_AWARE)."""
    benefit = min(deficit_pages, max(1, len(s.host_pages) or len(s.gpu_pages)))
    cost = max(1, s.context_len)
    return (Fraction(-benefit, cost), s.global_idx)


def compute_boundary_decisions(seqs: Seq[Sequence], eos_token_id: int, free_gpu_pages: Dict[int, int],
                               free_host_pages: int, buf: PageBufferConfig, kv_token_budget: int,
                               max_rows_per_bucket: int, host_chunk_tokens: int = 8192,
                               host_tier: bool = False, reclaimable_host_pages: int = 0) -> BoundaryDecisions:
    d = BoundaryDecisions()
    active: List[Sequence] = []
    for s in seqs:
        if s.status != S.IN_DECODE:
            continue
        if s.is_finished(eos_token_id):
            d.completed.append(s.global_idx)
        else:
            active.append(s)
    freed_gpu: Dict[int, int] = {}
    for s in seqs:
        if s.global_idx in d.completed:
            freed_gpu[s.decode_dp_group] = freed_gpu.get(s.decode_dp_group, 0) + len(s.gpu_pages)
    # ---- host growth + growth-driven eviction
    if host_tier:
        debt: Dict[int, int] = {}
        for s in active:
            if s.host_token_capacity - s.context_len <= buf.extension_gpu_page_buffer * buf.page_size:
                debt[s.global_idx] = pages_for(host_chunk_tokens, buf.page_size)
        need = sum(debt.values())
        supply = free_host_pages + sum(len(s.host_pages) for s in seqs if s.global_idx in d.completed)
        supply += reclaimable_host_pages
        if need > supply:
            victims = sorted((s for s in seqs if s.status in (S.PREFILLED, S.ON_HOLD, S.IN_DECODE)
                              and s.global_idx not in d.completed),
                             key=lambda s: _victim_key(s, need - supply))
            for v in victims:
                if need <= supply:
                    break
                supply += len(v.host_pages)
                need -= debt.pop(v.global_idx, 0)
                d.evicted.append(v.global_idx)
            if need > supply:
                d.scheduler_error = "[SCHED_INVARIANT] host KV growth infeasible after evicting every candidate"
        d.host_growth = debt
        active = [s for s in active if s.global_idx not in d.evicted]
    # ---- GPU extension or ON_HOLD per bucket
    by_bucket: Dict[int, List[Sequence]] = {}
    for s in active:
        by_bucket.setdefault(s.decode_dp_group, []).append(s)
    for b, rows in by_bucket.items():
        extra = {s.global_idx: extra_gpu_pages_needed(s.context_len, len(s.gpu_pages), buf, kv_token_budget)
                 for s in rows}
        free = free_gpu_pages.get(b, 0) + freed_gpu.get(b, 0)
        total = sum(extra.values())
        if total > free:
            order = sorted(rows, key=lambda s: (s.priority == Priority.HIGH, s.num_decoded, s.global_idx))
            for s in order:
                if total <= free:
                    break
                d.on_hold.append(s.global_idx)
                total -= extra.pop(s.global_idx)
                free += len(s.gpu_pages)
        d.extend.update({k: v for k, v in extra.items() if v > 0})
        free_after = free - sum(extra.values())
        # ---- load new rows into the freed space, most-decoded first
        slots = max_rows_per_bucket - (len(rows) - sum(1 for s in rows if s.global_idx in d.on_hold))
        cands = sorted((s for s in seqs if s.status in (S.PREFILLED, S.ON_HOLD) and s.decode_dp_group == b
                        and s.global_idx not in d.evicted and s.global_idx not in d.on_hold),
                       key=lambda s: (-s.num_decoded, s.global_idx))
        for s in cands:
            if slots <= 0:
                break
            need = gpu_pages_first_load(s.context_len, buf, kv_token_budget) - len(s.gpu_pages)
            need = max(0, need)
            if need <= free_after:
                free_after -= need
                slots -= 1
                d.load.append(s.global_idx)
    d.host_growth = {k: v for k, v in d.host_growth.items() if k not in d.on_hold}
    # buckets with no active rows can still load
    empty_buckets = set(free_gpu_pages) - set(by_bucket)
    for b in sorted(empty_buckets):
        free_after = free_gpu_pages[b] + freed_gpu.get(b, 0)
        slots = max_rows_per_bucket
        cands = sorted((s for s in seqs if s.status in (S.PREFILLED, S.ON_HOLD) and s.decode_dp_group == b
                        and s.global_idx not in d.evicted),
                       key=lambda s: (-s.num_decoded, s.global_idx))
        for s in cands:
            if slots <= 0:
                break
            need = max(0, gpu_pages_first_load(s.context_len, buf, kv_token_budget) - len(s.gpu_pages))
            if need <= free_after:
                free_after -= need
                slots -= 1
                d.load.append(s.global_idx)
    return d


def watermark_trigger(free_frac_per_node: Seq[float], watermark_pct: int, has_queued: bool,
                      has_evicted: bool) -> bool:
    """Leave decode for another prefill wave when host KV is under-used and work is waiting."""
    return max(free_frac_per_node) * 100.0 > watermark_pct and (has_queued or has_evicted)


def plan_kv_migration(used_pages_per_node: Seq[int], movable: Dict[int, List[Tuple[int, int]]],
                      ranks_per_node: int) -> List[Tuple[int, int, int, int]]:
    """Move the smallest parked rows from the most- to the least-loaded node until loads are within
    one row of the mean.  movable[node] = [(global_idx, pages)].  Returns
    [(global_idx, src_node, dst_node, dst_rank)] with destination ranks round-robin."""
    used = list(used_pages_per_node)
    n = len(used)
    if n <= 1:
        return []
    target = sum(used) / n
    pools = {k: sorted(v, key=lambda t: (t[1], t[0])) for k, v in movable.items()}
    rr = [0] * n
    plan = []
    for _ in range(10000):
        src = max(range(n), key=lambda i: (used[i], -i))
        dst = min(range(n), key=lambda i: (used[i], i))
        if not pools.get(src) or used[src] - target <= 0:
            break
        gid, pages = pools[src][0]
        if used[src] - pages < target - pages / 2 or used[dst] + pages > used[src] - pages + 2 * pages:
            if used[dst] + pages >= used[src]:
                break
        pools[src].pop(0)
        used[src] -= pages
        used[dst] += pages
        plan.append((gid, src, dst, dst * ranks_per_node + rr[dst] % ranks_per_node))
        rr[dst] += 1
    return plan


def plan_cohort_handover(stats: Dict[int, Dict[str, int]], in_flight: Seq[int] = ()) -> Optional[Tuple[int, int, int]]:
    """Data-parallel cohorts with separate engines: when one cohort has rows parked in its host tier (its device pool
    is full) while another is idle, hand half of the parked rows (at least one) to the idle cohort.
    ``stats[cohort]`` holds the last heartbeat's ``parked`` (rows that can move), ``live`` (sequences in the engine)
    and ``host_free`` (free host pages); cohorts in ``in_flight`` already take part in a hand-over.
    Returns (source, destination, rows) or None."""
    busy = set(in_flight)
    src = max((c for c in stats if c not in busy and stats[c].get("parked", 0) > 0),
              key=lambda c: (stats[c]["parked"], -c), default=None)
    if src is None:
        return None
    idle = [c for c in stats if c != src and c not in busy and stats[c].get("live", 0) == 0 and stats[c].get("host_free", 0) > 0]
    if not idle:
        return None
    dst = max(idle, key=lambda c: (stats[c]["host_free"], -c))
    return src, dst, max(1, stats[src]["parked"] // 2)
