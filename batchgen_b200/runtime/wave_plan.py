"""In-wave prefix sharing: plan one prefill wave so that every prefix shared inside the wave is computed once.

A wave is known in full before prefill starts, so the prefix tree of its prompts can be built from token ids
alone.  Prompts are cut into blocks of one KV page; the block that holds a prompt's last token is never
shared (it produces the first output token).  Runs of tree blocks that the same set of prompts passes
through form *segments*; a segment shared by at least ``threshold`` (>= 2) prompts is *pooled*: one item
computes it into the rank's prefix pool, every member reads it as an already-computed prefix.  Counts never
grow from a segment to its children, so the pooled set is closed under ancestors.  A prompt that continues a
committed trajectory can instead carry a *materialized* prefix: same geometry, but the pages are loaded from
the host KV tier and nobody computes them.

The planner is pure (no GPU, no host KV): it returns segments, work items, and chunks of items in an order
where an item only runs after all of its ancestor segments are resident.  The accounting identity

    prompt_tokens == computed_tokens + sum((members - 1) * tokens over computed segments)
                                     + sum( members      * tokens over materialized segments)

is checked by ``validate_wave_prefix_plan``.

``pack_wave_ranks`` spreads a wave over ranks: a prefix family stays on one rank (each rank owns its pool)
unless splitting it lowers the predicted makespan under a linear cost model
``sec = a + b*tokens/1e5 + c*attn_pairs/1e9 + d*rows/100 + e*chunks``; without a fitted profile it falls
back to balancing the sum of squared lengths.

Reference parity: batchgen/prefix_reuse/wave_plan.py:1-52 (definitions, accounting), :665
(plan_wave_prefix_sharing), :879 (validate); rank_packing.py:1-30,496 (pack_wave_ranks);
executor_cost.py:22-58 (cost model features).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

DECLINED_POOL_CHAIN_LONGER = "in_wave_pool_chain_longer_than_frontier"
DECLINED_DOES_NOT_FIT = "pool_materialization_does_not_fit"


@dataclass(frozen=True)
class MaterializedPrefix:
    index: int           # wave index of the prompt
    tokens: int          # page-aligned length of the committed prefix (>= one block, last token stays private)


@dataclass(frozen=True)
class PlanSegment:
    segment_id: int
    parent_id: Optional[int]        # nearest pooled ancestor
    token_start: int
    token_end: int
    members: Tuple[int, ...]
    materialized: bool = False

    @property
    def tokens(self) -> int:
        return self.token_end - self.token_start


@dataclass(frozen=True)
class PlanItem:
    kind: str                        # "segment" | "tail" | "materialize"
    ref: int                         # segment id, or wave index for a tail
    token_start: int
    token_end: int
    prefix_segments: Tuple[int, ...]  # pooled chain read as the computed prefix [0, token_start)

    @property
    def tokens(self) -> int:
        return 0 if self.kind == "materialize" else self.token_end - self.token_start


@dataclass
class WavePrefixPlan:
    block_tokens: int
    threshold: int
    segments: List[PlanSegment]
    items: List[PlanItem]
    chunks: List[List[int]]                         # indices into ``items``, in execution order
    release_after_chunk: Dict[int, int]             # segment id -> last chunk that reads it
    prompt_tokens: int
    computed_tokens: int
    peak_pool_pages: int
    declined_materialized: Dict[int, str] = field(default_factory=dict)

    @property
    def saved_tokens(self) -> int:
        return self.prompt_tokens - self.computed_tokens


class _Node:
    __slots__ = ("children", "members", "depth", "parent", "key")

    def __init__(self, depth: int, parent, key):
        self.children: Dict[bytes, "_Node"] = {}
        self.members: List[int] = []
        self.depth, self.parent, self.key = depth, parent, key


def _block_key(tokens: Sequence[int]) -> bytes:
    return hashlib.blake2b(b"".join(int(t).to_bytes(4, "little", signed=True) for t in tokens), digest_size=16).digest()


def _build_tree(prompts: Sequence[Sequence[int]], block: int, skip: Sequence[int]) -> _Node:
    root = _Node(0, None, None)
    skipset = set(skip)
    for i, p in enumerate(prompts):
        if i in skipset:
            continue
        node = root
        for b in range((len(p) - 1) // block):
            key = _block_key(p[b * block:(b + 1) * block])
            nxt = node.children.get(key)
            if nxt is None:
                nxt = node.children[key] = _Node(node.depth + 1, node, key)
            nxt.members.append(i)
            node = nxt
    return root


def _segments(root: _Node, block: int, threshold: int) -> List[PlanSegment]:
    """Maximal runs with an unchanged member set, kept when pooled; parents precede children."""
    out: List[PlanSegment] = []
    stack = [(child, None) for child in root.children.values()]
    while stack:
        start, parent_seg = stack.pop()
        if len(start.members) < max(2, threshold):
            continue                                   # counts are monotone: nothing below is pooled either
        end = start
        while len(end.children) == 1:
            (only,) = end.children.values()
            if len(only.members) != len(end.members):
                break
            end = only
        sid = len(out)
        out.append(PlanSegment(sid, parent_seg, (start.depth - 1) * block, end.depth * block, tuple(start.members)))
        stack.extend((c, sid) for c in end.children.values())
    return out


def plan_wave_prefix_sharing(prompts: Sequence[Sequence[int]], block_tokens: int, threshold: int = 2,
                             chunk_tokens: int = 131072, pool_pages: Optional[int] = None,
                             materialized: Sequence[MaterializedPrefix] = ()) -> WavePrefixPlan:
    """Plan one wave.  ``pool_pages`` bounds the pages resident in the prefix pool at any time: the
    threshold is raised (fewer, more valuable segments) until the schedule fits, and materialized hits that
    still do not fit are declined by name."""
    if block_tokens <= 0:
        raise ValueError("block_tokens must be positive")
    threshold = max(2, threshold)
    # ---- which materialized hits to keep: only if at least as long as the row's best in-wave pool chain
    declined: Dict[int, str] = {}
    keep: List[MaterializedPrefix] = []
    if materialized:
        probe = _segments(_build_tree(prompts, block_tokens, ()), block_tokens, threshold)
        best_chain = {}
        for s in probe:
            for m in s.members:
                best_chain[m] = max(best_chain.get(m, 0), s.token_end)
        for hit in sorted(materialized, key=lambda h: -h.tokens):
            limit = ((len(prompts[hit.index]) - 1) // block_tokens) * block_tokens
            if hit.tokens % block_tokens or hit.tokens <= 0 or hit.tokens > limit:
                raise ValueError(f"materialized prefix of prompt {hit.index} must be page aligned, non-empty and "
                                 "leave the last token private")
            if best_chain.get(hit.index, 0) > hit.tokens:
                declined[hit.index] = DECLINED_POOL_CHAIN_LONGER
            else:
                keep.append(hit)
    while True:
        plan = _plan_once(prompts, block_tokens, threshold, chunk_tokens, keep)
        if pool_pages is None or plan.peak_pool_pages <= pool_pages:
            break
        if any(len(s.members) >= threshold and not s.materialized for s in plan.segments):
            counts = sorted({len(s.members) for s in plan.segments if not s.materialized})
            threshold = next((c + 1 for c in counts if c >= threshold), threshold + 1)
            continue
        if keep:                                       # only loaded prefixes are left: drop the smallest
            drop = keep.pop()
            declined[drop.index] = DECLINED_DOES_NOT_FIT
            continue
        break
    plan.declined_materialized = declined
    return plan


def _plan_once(prompts, block, threshold, chunk_tokens, keep: Sequence[MaterializedPrefix]) -> WavePrefixPlan:
    mat_rows = {h.index: h for h in keep}
    root = _build_tree(prompts, block, list(mat_rows))
    segs = _segments(root, block, threshold)
    for h in keep:
        segs.append(PlanSegment(len(segs), None, 0, h.tokens, (h.index,), materialized=True))
    chain: Dict[int, List[int]] = {i: [] for i in range(len(prompts))}
    for s in segs:                                      # parents precede children -> chains are root-first
        for m in s.members:
            chain[m].append(s.segment_id)
    # ---- items in depth-first order: a segment, then everything below it, so pools drain early
    children: Dict[Optional[int], List[int]] = {}
    for s in segs:
        children.setdefault(s.parent_id, []).append(s.segment_id)
    tails_under: Dict[Optional[int], List[int]] = {}
    for i in range(len(prompts)):
        tails_under.setdefault(chain[i][-1] if chain[i] else None, []).append(i)
    items: List[PlanItem] = []

    def prefix_of(seg: Optional[int]) -> Tuple[int, ...]:
        out = []
        while seg is not None:
            out.append(seg)
            seg = segs[seg].parent_id
        return tuple(reversed(out))

    def emit(seg: Optional[int]) -> None:
        for i in sorted(tails_under.get(seg, [])):
            start = segs[seg].token_end if seg is not None else 0
            items.append(PlanItem("tail", i, start, len(prompts[i]), prefix_of(seg)))
        for c in sorted(children.get(seg, []), key=lambda c: -len(segs[c].members)):
            s = segs[c]
            items.append(PlanItem("materialize" if s.materialized else "segment", c, s.token_start, s.token_end,
                                  prefix_of(s.parent_id)))
            emit(c)

    emit(None)
    # ---- chunks: token budget; an item and the segment it reads may share a chunk only if the segment's item
    #      comes earlier in the same chunk (the prepacked forward treats earlier rows' pages as written)
    chunks: List[List[int]] = [[]]
    used = 0
    for idx, it in enumerate(items):
        if it.tokens and used + it.tokens > chunk_tokens and chunks[-1]:
            chunks.append([])
            used = 0
        chunks[-1].append(idx)
        used += it.tokens
    if not chunks[-1]:
        chunks.pop()
    # ---- residency: a segment is released after the last chunk with an item that reads or writes it
    release: Dict[int, int] = {}
    for ci, ch in enumerate(chunks):
        for idx in ch:
            it = items[idx]
            for sid in it.prefix_segments + ((it.ref,) if it.kind != "tail" else ()):
                release[sid] = ci
    first_chunk = {}
    for ci, ch in enumerate(chunks):
        for idx in ch:
            it = items[idx]
            if it.kind != "tail":
                first_chunk.setdefault(it.ref, ci)
    peak = 0
    for ci in range(len(chunks)):
        live = sum(-(-segs[sid].tokens // block) for sid in release if first_chunk.get(sid, 0) <= ci <= release[sid])
        peak = max(peak, live)
    prompt_tokens = sum(len(p) for p in prompts)
    computed = sum(it.tokens for it in items)
    return WavePrefixPlan(block, threshold, segs, items, chunks, release, prompt_tokens, computed, peak)


def validate_wave_prefix_plan(plan: WavePrefixPlan, prompts: Sequence[Sequence[int]]) -> None:
    """Raise ``ValueError`` naming the first broken invariant."""
    segs = {s.segment_id: s for s in plan.segments}
    saved = sum((len(s.members) - (0 if s.materialized else 1)) * s.tokens for s in plan.segments)
    if plan.prompt_tokens != plan.computed_tokens + saved:
        raise ValueError(f"accounting: {plan.prompt_tokens} != {plan.computed_tokens} + {saved}")
    done = set()
    tails = set()
    for ch in plan.chunks:
        for idx in ch:
            it = plan.items[idx]
            for sid in it.prefix_segments:
                if sid not in done:
                    raise ValueError(f"item {idx} reads segment {sid} before it is resident")
            expect = 0
            for sid in it.prefix_segments:
                if segs[sid].token_start != expect:
                    raise ValueError(f"item {idx}: prefix chain has a gap at token {expect}")
                expect = segs[sid].token_end
            if it.token_start != expect:
                raise ValueError(f"item {idx} starts at {it.token_start}, its prefix ends at {expect}")
            if it.kind == "tail":
                if it.token_end != len(prompts[it.ref]) or it.token_end <= it.token_start:
                    raise ValueError(f"tail of prompt {it.ref} must end at the prompt end and hold its last token")
                tails.add(it.ref)
            else:
                s = segs[it.ref]
                for m in s.members:
                    if list(prompts[m][s.token_start:s.token_end]) != list(prompts[s.members[0]][s.token_start:s.token_end]):
                        raise ValueError(f"segment {s.segment_id}: member {m} does not share its tokens")
                done.add(it.ref)
    if tails != set(range(len(prompts))):
        raise ValueError("every prompt needs exactly one tail item")


# ------------------------------------------------------------------------------------------------ rank packing
@dataclass(frozen=True)
class CostProfile:
    """sec = a + b*tokens/1e5 + c*attn_pairs/1e9 + d*rows/100 + e*chunks, fitted per (model, GPU, group size)."""
    a: float = 0.0
    b: float = 1.0
    c: float = 1.0
    d: float = 0.0
    e: float = 0.0

    def seconds(self, tokens: int, attn_pairs: int, rows: int, chunks: int) -> float:
        return self.a + self.b * tokens / 1e5 + self.c * attn_pairs / 1e9 + self.d * rows / 100 + self.e * chunks


_PROFILES: Dict[Tuple[str, str, int], CostProfile] = {}


def register_cost_profile(model: str, gpu: str, group_size: int, profile: CostProfile) -> None:
    _PROFILES[(model, gpu, group_size)] = profile


def find_cost_profile(model: str, gpu: str, group_size: int) -> Optional[CostProfile]:
    """No fallback across models or GPUs: an unfitted combination returns None (callers balance L^2 instead)."""
    return _PROFILES.get((model, gpu, group_size))


def _tri(n: int) -> int:
    return n * (n + 1) // 2


def _unit_features(prompts, members: Sequence[int], block: int, chunk_tokens: int) -> Tuple[int, int, int, int]:
    """(computed tokens, causal attention pairs, rows, chunks) of a set of prompts prefilled on one rank."""
    sub = [prompts[i] for i in members]
    plan = plan_wave_prefix_sharing(sub, block, 2, chunk_tokens)
    pairs = sum(_tri(it.token_end) - _tri(it.token_start) for it in plan.items if it.kind != "materialize")
    rows = sum(1 for it in plan.items if it.kind != "materialize")
    return plan.computed_tokens, pairs, rows, len(plan.chunks)


@dataclass
class RankPacking:
    rank_of: List[int]                 # wave index -> rank
    predicted: List[float]             # per-rank score (seconds under a profile, else sum of L^2)
    digest: str                        # identical on every rank for identical inputs

    @property
    def makespan(self) -> float:
        return max(self.predicted) if self.predicted else 0.0


def pack_wave_ranks(prompts: Sequence[Sequence[int]], n_ranks: int, block_tokens: int, chunk_tokens: int = 131072,
                    profile: Optional[CostProfile] = None, rounds: int = 14,
                    initial_load: Optional[Sequence[float]] = None) -> RankPacking:
    """Families (prompts sharing their first block) stay together; the heaviest family on the slowest rank
    is split in two while that lowers the predicted makespan (at most ``rounds`` refinements).  ``initial_load``
    is what each rank already carries, in the unit of the score (sum of squared lengths without a profile)."""
    fam: Dict[bytes, List[int]] = {}
    for i, p in enumerate(prompts):
        key = _block_key(p[:block_tokens]) if len(p) > block_tokens else b"solo%d" % i
        fam.setdefault(key, []).append(i)
    units: List[List[int]] = list(fam.values())

    def score(members: Sequence[int]) -> float:
        if profile is None:
            return float(sum(len(prompts[i]) ** 2 for i in members))
        return profile.seconds(*_unit_features(prompts, members, block_tokens, chunk_tokens))

    def place(us: List[List[int]]):
        load = [float(v) for v in initial_load] if initial_load is not None else [0.0] * n_ranks
        where: List[int] = []
        order = sorted(range(len(us)), key=lambda u: -score(us[u]))
        where = [0] * len(us)
        for u in order:
            r = min(range(n_ranks), key=lambda r: (load[r], r))
            where[u] = r
            load[r] += score(us[u])
        return where, load

    where, load = place(units)
    for _ in range(rounds):
        worst = max(range(n_ranks), key=lambda r: load[r])
        cands = [u for u in range(len(units)) if where[u] == worst and len(units[u]) > 1]
        if not cands:
            break
        u = max(cands, key=lambda u: score(units[u]))
        mem = sorted(units[u], key=lambda i: -len(prompts[i]))
        trial = units[:u] + units[u + 1:] + [mem[0::2], mem[1::2]]
        w2, l2 = place(trial)
        if max(l2) + 1e-12 < max(load):
            units, where, load = trial, w2, l2
        else:
            break
    rank_of = [0] * len(prompts)
    for u, members in enumerate(units):
        for i in members:
            rank_of[i] = where[u]
    digest = hashlib.blake2b(",".join(map(str, rank_of)).encode(), digest_size=8).hexdigest()
    return RankPacking(rank_of, load, digest)


def first_divergence(digests: Sequence[str], packings: Sequence[Sequence[int]]) -> Optional[int]:
    """Cross-check of a packing gathered from every rank: index of the first prompt whose rank differs."""
    if len(set(digests)) <= 1:
        return None
    base = packings[0]
    for i in range(len(base)):
        if any(p[i] != base[i] for p in packings[1:]):
            return i
    return None
