"""Moving parked sequences between data-parallel ranks: the executor of ``scheduler.plan_kv_migration``.

A row that is on hold keeps its KV in the host tier (and, for models with KDA layers, its recurrent state in the
host state store).  When the nodes' host tiers fill unevenly, the planner picks rows to move; this module ships
one: a small header (token ids, sampling parameters, counters) and the host pages, layer-major, over
``torch.distributed`` point-to-point (NCCL between GPU boxes, gloo on CPU).  The source frees its pages and
forgets the row; the destination allocates pages, registers the row as ON_HOLD and resumes it like any other
parked row, so the tokens produced are the ones the source would have produced.

Reference parity: host-KV migration between DP ranks at decode boundaries
(batchgen/scheduler.py kv-migration planning, batchgen/batchgen.py migration step).
"""
from __future__ import annotations

import dataclasses
import json
from typing import List, Sequence as Seq, Tuple

import torch
import torch.distributed as dist

from .sequence import S, SamplingParams, Sequence


def _pack_header(s: Sequence, n_pages: int, has_state: bool) -> torch.Tensor:
    d = {"global_idx": s.global_idx, "prompt_ids": s.prompt_ids, "output_ids": s.output_ids,
         "params": dataclasses.asdict(s.params), "custom_id": s.custom_id, "batch_id": s.batch_id,
         "num_cached_tokens": s.num_cached_tokens, "cached_prefix_tokens": s.cached_prefix_tokens,
         "total_decoded_before_eviction": s.total_decoded_before_eviction,
         "had_initial_gpu_reservation": s.had_initial_gpu_reservation, "n_pages": n_pages, "has_state": has_state}
    return torch.frombuffer(bytearray(json.dumps(d).encode()), dtype=torch.uint8).clone()


def send_sequence(engine, s: Sequence, dst: int, group=None) -> int:
    """Ship a row that is ON_HOLD in the host tier to rank ``dst``; returns the bytes sent.  The row leaves
    this engine (pages and state item freed)."""
    if s.status != S.ON_HOLD or not s.host_pages or s.gpu_pages:
        raise ValueError(f"seq {s.global_idx} is not parked in the host tier")
    hk = engine.host_kv
    has_state = s.state_item >= 0
    hdr = _pack_header(s, len(s.host_pages), has_state)
    dist.send(torch.tensor([hdr.numel()], dtype=torch.int64), dst, group=group)
    dist.send(hdr, dst, group=group)
    pages = torch.as_tensor(s.host_pages, dtype=torch.long)
    kv = hk.kv[:, pages].contiguous()
    dist.send(kv, dst, group=group)
    sent = hdr.numel() + kv.numel() * kv.element_size()
    if hk.idx_k is not None:
        ik, isc = hk.idx_k.view(torch.uint8)[:, pages].contiguous(), hk.idx_s[:, pages].contiguous()
        dist.send(ik, dst, group=group)
        dist.send(isc, dst, group=group)
        sent += ik.numel() + isc.numel() * 4
    if has_state:
        hs = engine.host_state
        rec, conv = hs.rec[:, s.state_item].contiguous(), hs.conv[:, s.state_item].contiguous()
        dist.send(rec, dst, group=group)
        dist.send(conv, dst, group=group)
        sent += (rec.numel() + conv.numel()) * 4
        hs.release(s.state_item)
        s.state_item = -1
    hk.alloc.free(s.host_pages)
    s.host_pages = []
    del engine.seqs[s.global_idx]
    return sent


def recv_sequence(engine, src: int, group=None) -> Sequence:
    """Counterpart of ``send_sequence``: allocate host pages, receive the row and register it as ON_HOLD."""
    n = torch.zeros(1, dtype=torch.int64)
    dist.recv(n, src, group=group)
    hdr = torch.zeros(int(n), dtype=torch.uint8)
    dist.recv(hdr, src, group=group)
    d = json.loads(bytes(hdr.tolist()).decode())
    hk = engine.host_kv
    if d["global_idx"] in engine.seqs:
        raise ValueError(f"seq {d['global_idx']} already lives here")
    pages = hk.alloc.alloc(d["n_pages"])
    idx = torch.as_tensor(pages, dtype=torch.long)
    kv = torch.empty(hk.kv.shape[0], len(pages), *hk.kv.shape[2:], dtype=hk.kv.dtype)
    dist.recv(kv, src, group=group)
    hk.kv[:, idx] = kv
    if hk.idx_k is not None:
        ik = torch.empty(hk.idx_k.shape[0], len(pages), *hk.idx_k.shape[2:], dtype=torch.uint8)
        isc = torch.empty(hk.idx_s.shape[0], len(pages), *hk.idx_s.shape[2:], dtype=hk.idx_s.dtype)
        dist.recv(ik, src, group=group)
        dist.recv(isc, src, group=group)
        hk.idx_k.view(torch.uint8)[:, idx] = ik
        hk.idx_s[:, idx] = isc
    s = Sequence(global_idx=d["global_idx"], prompt_ids=d["prompt_ids"], params=SamplingParams(**d["params"]),
                 custom_id=d["custom_id"], batch_id=d["batch_id"])
    s.output_ids = list(d["output_ids"])
    s.num_cached_tokens = d["num_cached_tokens"]
    s.cached_prefix_tokens = d["cached_prefix_tokens"]
    s.total_decoded_before_eviction = d["total_decoded_before_eviction"]
    s.had_initial_gpu_reservation = d["had_initial_gpu_reservation"]
    s.host_pages = pages
    if d["has_state"]:
        hs = engine.host_state
        if hs is None:
            raise RuntimeError("the destination keeps no host state store")
        item = hs.reserve()
        rec, conv = torch.empty_like(hs.rec[:, item]), torch.empty_like(hs.conv[:, item])
        dist.recv(rec, src, group=group)
        dist.recv(conv, src, group=group)
        hs.rec[:, item] = rec
        hs.conv[:, item] = conv
        s.state_item = item
    s.status = S.ON_HOLD
    s.history.append(f"migrated from rank {src}")
    s.assigned_rank = dist.get_rank(group)
    engine.seqs[s.global_idx] = s
    engine._next_idx = max(engine._next_idx, s.global_idx + 1)
    return s


def execute_plan(engine, plan: Seq[Tuple[int, int, int, int]], rank: int, holder_rank=None, group=None) -> int:
    """Run the entries of a ``plan_kv_migration`` result that involve this rank, in plan order (every rank
    walks the same list, so sends and receives pair up).  ``holder_rank(global_idx, src_node)`` names the rank
    that holds a row (default: one rank per node, the node index).  Returns the rows moved in or out."""
    holder_rank = holder_rank or (lambda gid, node: node)
    moved = 0
    for gid, src_node, dst_node, dst_rank in plan:
        src = holder_rank(gid, src_node)
        if src == dst_rank:
            continue
        if rank == src:
            send_sequence(engine, engine.seqs[gid], dst_rank, group)
            moved += 1
        elif rank == dst_rank:
            recv_sequence(engine, src, group)
            moved += 1
    return moved


# ---------------------------------------------------------------------------------------------------------------
# Hand-over between engines that share no process group (the server's data-parallel cohorts): a parked row is
# packed into one payload (header + tensors), travels as a file or any other byte channel, and is adopted by
# another engine under a fresh sequence number of that engine.
def can_export(engine) -> bool:
    hk = getattr(engine, "host_kv", None)
    return hk is not None and getattr(hk, "kv", None) is not None and not engine.cfg.is_v4


def export_sequence(engine, s: Sequence) -> dict:
    """Pack a row that is ON_HOLD in the host tier and remove it from ``engine``."""
    if s.status != S.ON_HOLD or not s.host_pages or s.gpu_pages:
        raise ValueError(f"seq {s.global_idx} is not parked in the host tier")
    hk = engine.host_kv
    if not can_export(engine):
        raise NotImplementedError("hand-over covers the paged latent / GQA KV of the torch host tier")
    pages = torch.as_tensor(s.host_pages, dtype=torch.long)
    has_state = s.state_item >= 0
    payload = {"header": json.loads(bytes(_pack_header(s, len(s.host_pages), has_state).tolist()).decode()),
               "kv": hk.kv[:, pages].clone()}
    payload["header"]["session_id"] = s.session_id
    if hk.idx_k is not None:
        payload["idx_k"] = hk.idx_k.view(torch.uint8)[:, pages].clone()
        payload["idx_s"] = hk.idx_s[:, pages].clone()
    if has_state:
        hs = engine.host_state
        payload["rec"], payload["conv"] = hs.rec[:, s.state_item].clone(), hs.conv[:, s.state_item].clone()
        hs.release(s.state_item)
        s.state_item = -1
    hk.alloc.free(s.host_pages)
    s.host_pages = []
    del engine.seqs[s.global_idx]
    return payload


def import_sequence(engine, payload: dict, assigned_rank: int = 0) -> Sequence:
    """Adopt a packed row: host pages are allocated here, the row becomes ON_HOLD under this engine's next sequence
    number and resumes like any other parked row.  Raises ``OutOfPages`` when the host tier has no room."""
    d = payload["header"]
    hk = engine.host_kv
    if hk is None:
        raise RuntimeError("the destination keeps no host tier")
    pages = hk.alloc.alloc(d["n_pages"])
    idx = torch.as_tensor(pages, dtype=torch.long)
    hk.kv[:, idx] = payload["kv"].to(hk.kv.dtype)
    if hk.idx_k is not None and "idx_k" in payload:
        hk.idx_k.view(torch.uint8)[:, idx] = payload["idx_k"]
        hk.idx_s[:, idx] = payload["idx_s"]
    s = Sequence(global_idx=engine._next_idx, prompt_ids=d["prompt_ids"], params=SamplingParams(**d["params"]),
                 custom_id=d["custom_id"], batch_id=d["batch_id"])
    engine._next_idx += 1
    s.output_ids = list(d["output_ids"])
    s.num_cached_tokens = d["num_cached_tokens"]
    s.cached_prefix_tokens = d["cached_prefix_tokens"]
    s.total_decoded_before_eviction = d["total_decoded_before_eviction"]
    s.had_initial_gpu_reservation = d["had_initial_gpu_reservation"]
    s.session_id = d.get("session_id")
    s.host_pages = pages
    if d["has_state"]:
        hs = engine.host_state
        if hs is None:
            raise RuntimeError("the destination keeps no host state store")
        item = hs.reserve()
        hs.rec[:, item] = payload["rec"]
        hs.conv[:, item] = payload["conv"]
        s.state_item = item
    s.status = S.ON_HOLD
    s.history.append("adopted from another engine")
    s.assigned_rank = assigned_rank
    engine.seqs[s.global_idx] = s
    return s


def parked_rows(engine) -> List[Sequence]:
    """Rows that can be handed over right now: on hold, KV entirely in the host tier, no step in flight; smallest first.
    Empty when this engine's host tier cannot be packed by ``export_sequence`` (the native region, whose rows would move
    by page ownership instead, and the DeepSeek-V4 pools)."""
    if not can_export(engine):
        return []
    rows = [s for s in engine.seqs.values()
            if s.status == S.ON_HOLD and s.host_pages and not s.gpu_pages and not getattr(s, "inflight_tokens", 0)]
    return sorted(rows, key=lambda s: (len(s.host_pages), s.global_idx))
