"""Serve groups for DP(world / G) x TP-G resident decode.

With tensor-parallel attention over G ranks the world splits into ``world // G`` groups of contiguous
ranks.  A sequence binds to one group at admission and every rank of the group holds it (replicated
attention rows, head-sharded state), so membership must resolve identically on all G ranks:
``seq.decode_dp_group == rank // G``.  The node-shared host KV entry of a sequence is touched by exactly one
rank, the group leader ``g * G``.  G == 1 collapses to pure DP (group id == rank).

Everything here is pure arithmetic so that it can be tested without GPUs.

Reference parity: batchgen/decode_dp_group.py:52-160 (group count, membership, owner, eviction memory,
FFD assignment), :161-260 (plan digest, disagreement check, MoE rows per rank).
"""
from __future__ import annotations

import hashlib
import math
from typing import Iterable, List, Optional, Sequence, Tuple


def num_decode_dp_groups(world_size: int, group_size: int) -> int:
    if group_size <= 0 or world_size % group_size:
        raise ValueError(f"group_size {group_size} must be positive and divide world_size {world_size}")
    return world_size // group_size


def rank_in_decode_group(decode_dp_group: Optional[int], global_rank: int, group_size: int) -> bool:
    if decode_dp_group is None:
        return False
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    return int(decode_dp_group) == global_rank // group_size


def host_kv_owner_rank(decode_dp_group: int, group_size: int) -> int:
    """The one rank that registers / grows / releases a group's sequences in the node-shared host KV."""
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    return int(decode_dp_group) * group_size


def evict_from_decode_dp_group(seq) -> None:
    """Drop the group of an evicted sequence but remember it: its decoded tokens live in the trajectory
    book of that group's node, so the re-entry is pinned back to the same group."""
    if getattr(seq, "decode_dp_group", None) is not None:
        seq.evicted_from_dp_group = seq.decode_dp_group
    seq.decode_dp_group = None


def assign_decode_dp_groups(lengths: Sequence[int], num_dp: int, prior_load: Optional[Sequence[float]] = None,
                            use_l2: bool = True, pinned: Optional[Sequence[Optional[int]]] = None) -> List[int]:
    """Longest first onto the least-loaded group (load = sum of L^2, or count).  ``pinned[i]`` forces a
    group (re-entries after eviction) and still adds to that group's load."""
    if num_dp <= 0:
        raise ValueError("num_dp must be positive")
    if prior_load is not None and len(prior_load) != num_dp:
        raise ValueError("prior_load must have one entry per group")
    load = [float(x) for x in prior_load] if prior_load is not None else [0.0] * num_dp
    out = [0] * len(lengths)
    for i in sorted(range(len(lengths)), key=lambda i: (-(lengths[i] or 0), i)):
        L = float(lengths[i] or 0)
        if pinned is not None and pinned[i] is not None:
            g = int(pinned[i])
            if not 0 <= g < num_dp:
                raise ValueError(f"sequence {i} is pinned to group {g} of {num_dp}")
        else:
            g = min(range(num_dp), key=lambda r: (load[r], r))
        out[i] = g
        load[g] += L * L if use_l2 else 1.0
    return out


def decode_group_plan_digest(pairs: Sequence[Tuple[int, int]]) -> int:
    """64-bit digest of (global_idx, group) pairs; every rank must compute the same value."""
    h = hashlib.blake2b(digest_size=8)
    for gi, g in sorted(pairs):
        h.update(int(gi).to_bytes(8, "little", signed=True) + int(g).to_bytes(4, "little", signed=True))
    return int.from_bytes(h.digest(), "little")


def first_group_disagreement(plans: Sequence[Sequence[Tuple[int, int]]]) -> Optional[Tuple[int, List[Optional[int]]]]:
    """Given every rank's plan, the first global_idx whose group differs (and what each rank said)."""
    maps = [dict(p) for p in plans]
    for gi in sorted(set().union(*[m.keys() for m in maps]) if maps else []):
        vals = [m.get(gi) for m in maps]
        if len(set(vals)) > 1:
            return gi, vals
    return None


def moe_rows_per_rank(max_group_batch: int, group_size: int) -> int:
    """Rows each rank owns after a group's batch is scattered over its G ranks for the EP MoE."""
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    return int(math.ceil(int(max_group_batch) / group_size))


def decode_group_rows(rank_counts: Sequence[int], group_size: int) -> List[int]:
    if group_size <= 0 or len(rank_counts) % group_size:
        raise ValueError("rank counts must split into groups")
    c = [int(v) for v in rank_counts]
    return [max(c[s:s + group_size]) for s in range(0, len(c), group_size)]


def count_rows_per_group(group_ids: Iterable[Optional[int]], num_dp: int) -> List[int]:
    rows = [0] * num_dp
    for g in group_ids:
        if g is not None:
            rows[int(g)] += 1
    return rows
