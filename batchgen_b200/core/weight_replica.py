"""Weight replica planning: who copies a streamed module from host memory, and who pulls it from a peer.

When weights do not fit in HBM every rank streams the same modules (attention blocks, shared experts,
routed experts) through its GPU weight ring.  Ranks of one node that can reach each other over NVLink form a
*replica group*: each module is copied host->device by exactly one owner rank and the other members pull it
GPU->GPU from the owner's ring slot, so the PCIe traffic of the node is divided by the group size.

* ``compute_replica_groups``: group = ranks on the same node with the same module list and mutual peer
  access.  A partial peer-access matrix is an install error (no silent smaller clique).
* ``derive_frame_plan``: a pass is a sequence of *frames* (one per layer); each module type contributes a
  constant number of modules per frame (``routed_expert_<layer>_<expert>``, ``attn_<layer>``,
  ``shared_expert_<layer>``).  A task that does not fit this grammar gets no plan (single-member groups).
* ``derive_owner_map``: routed experts are owned in contiguous blocks, single-module types round-robin by
  layer, so every member copies the same number of bytes per frame.
* ``plan_broadcast_frames``: for a cross-node group the owner broadcasts staged slots in a canonical order
  that every member derives independently.

Reference parity: batchgen/weight_replica_group.py:153-183 (groups), :213-281 (frame plan), :283-308 (owner
map); batchgen/weight_replica_transport.py:96-170 (broadcast frame order);
core/GPU_Weight_Buffer/weight_replica_plan.h:60-85 (record kinds).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

HOST_PRIVATE, REPLICA_OWNER, REPLICA_READER = "host_private", "replica_owner", "replica_reader"


@dataclass(frozen=True)
class RankRecord:
    rank: int
    node_identity: str                 # ranks on different nodes never share a group
    list_fingerprint: str              # hash of the rank's ordered module list
    peer_access: Mapping[int, bool]    # rank -> can this rank read that rank's ring slots
    weight_source_kind: str = "host"   # "resident": the rank already holds everything, group of one


def compute_replica_groups(records: Sequence[RankRecord]) -> Dict[int, Tuple[int, ...]]:
    groups: Dict[int, Tuple[int, ...]] = {}
    buckets: Dict[Tuple[str, str], List[RankRecord]] = {}
    for r in records:
        if r.weight_source_kind == "resident":
            groups[r.rank] = (r.rank,)
        else:
            buckets.setdefault((r.node_identity, r.list_fingerprint), []).append(r)
    for members in buckets.values():
        members.sort(key=lambda r: r.rank)
        for a in members:
            for b in members:
                if a.rank != b.rank and not a.peer_access.get(b.rank, False):
                    raise ValueError(f"partial peer access inside a replica group: rank {a.rank} cannot read rank "
                                     f"{b.rank}; ranks {[m.rank for m in members]} share node and module list")
        g = tuple(m.rank for m in members)
        for m in members:
            groups[m.rank] = g
    return groups


_NAME = {"routed_expert": re.compile(r"^routed_expert_(\d+)_(\d+)$"), "attn": re.compile(r"^attn_(\d+)$"),
         "shared_expert": re.compile(r"^shared_expert_(\d+)$")}


def _parse(module_type: str, name: str) -> Optional[Tuple[int, Optional[int]]]:
    pat = _NAME.get(module_type)
    m = pat.match(name) if pat else None
    if not m:
        return None
    return (int(m.group(1)), int(m.group(2))) if module_type == "routed_expert" else (int(m.group(1)), None)


@dataclass(frozen=True)
class FramePlan:
    layer_sequence: Tuple[int, ...]
    frame_size: Dict[str, int]                           # modules of each type per frame
    position: Dict[str, Tuple[int, Optional[int]]]       # module -> (frame index, expert index or None)


def derive_frame_plan(task: Mapping[str, Sequence[str]]) -> Optional[FramePlan]:
    layers_of: Dict[str, List[int]] = {}
    size: Dict[str, int] = {}
    for mtype, names in task.items():
        if not names:
            continue
        layers: List[int] = []
        counts: List[int] = []
        for n in names:
            p = _parse(mtype, n)
            if p is None:
                return None
            if not layers or p[0] != layers[-1]:
                if layers and p[0] < layers[-1]:
                    return None                           # layers out of order
                layers.append(p[0])
                counts.append(0)
            counts[-1] += 1
        if len(set(counts)) != 1:
            return None                                   # ragged frames
        layers_of[mtype], size[mtype] = layers, counts[0]
    if not size:
        return None
    union = sorted({l for seq in layers_of.values() for l in seq})
    idx = {l: i for i, l in enumerate(union)}
    pos = {}
    for mtype, names in task.items():
        for n in names:
            layer, expert = _parse(mtype, n)
            pos[n] = (idx[layer], expert)
    return FramePlan(tuple(union), size, pos)


def derive_owner_map(group: Sequence[int], task: Mapping[str, Sequence[str]], plan: FramePlan) -> Dict[str, int]:
    owners: Dict[str, int] = {}
    g = list(group)
    for mtype, names in task.items():
        if not names:
            continue
        per_frame = plan.frame_size[mtype]
        for n in names:
            frame, expert = plan.position[n]
            if expert is None:
                owners[n] = g[frame % len(g)]
            else:
                if per_frame % len(g):
                    raise ValueError(f"{mtype}: {per_frame} modules per frame do not divide over {len(g)} replicas")
                # experts of one frame are numbered from the frame's first expert
                first = min(e for (f, e) in (plan.position[m] for m in names) if f == frame)
                owners[n] = g[(expert - first) // (per_frame // len(g))]
    return owners


def record_kinds(rank: int, group: Sequence[int], owners: Mapping[str, int]) -> Dict[str, str]:
    """What this rank does with each module: copy it from host and serve it, pull it from the owner, or (group
    of one) plain private copy."""
    if len(group) <= 1:
        return {n: HOST_PRIVATE for n in owners}
    return {n: (REPLICA_OWNER if o == rank else REPLICA_READER) for n, o in owners.items()}


def bytes_copied_per_rank(owners: Mapping[str, int], sizes: Mapping[str, int]) -> Dict[int, int]:
    out: Dict[int, int] = {}
    for n, o in owners.items():
        out[o] = out.get(o, 0) + int(sizes[n])
    return out


@dataclass(frozen=True)
class BroadcastFrame:
    frame: int
    owner: int
    modules: Tuple[str, ...]


def plan_broadcast_frames(task: Mapping[str, Sequence[str]], plan: FramePlan, owners: Mapping[str, int]
                          ) -> List[BroadcastFrame]:
    """Canonical broadcast order for a cross-node group: frames in pass order, inside a frame owners in rank
    order, inside an owner modules by (type, expert).  Every member derives the same list."""
    per: Dict[Tuple[int, int], List[Tuple[str, int, str]]] = {}
    for mtype in sorted(task):
        for n in task[mtype]:
            frame, expert = plan.position[n]
            per.setdefault((frame, owners[n]), []).append((mtype, -1 if expert is None else expert, n))
    out = []
    for (frame, owner) in sorted(per):
        out.append(BroadcastFrame(frame, owner, tuple(n for _, _, n in sorted(per[(frame, owner)]))))
    return out
