"""Whole-decode-step CUDA graphs with bucketed batch sizes.

One graph per bucket captures the entire model forward of a decode step (every layer: norms, FP8
GEMMs, MLA attention, router, dispatch, grouped expert GEMMs, combine — and, on multi-GPU jobs, the
fused NVLink kernels or the NCCL collectives between them).  Inputs live in static device buffers that
are refreshed from pinned host staging before each replay; rows past the real batch are padding
(``seqlens = 0``, ``slot = -1``, router told through a device-resident ``num_valid``), so a bucket's
graph serves every batch size up to the bucket.

The fused communication kernels take their epochs as *offset + device-resident base*, and the base is
bumped by a kernel at the end of each step, so replaying a graph publishes fresh epochs every time.

Reference parity: batchgen/cuda_graph/graph_manager.py:37-547 (segments x buckets, static buffers,
capture/replay, capture-memory ledger), buckets.py:13,99 (bucket generation), compare.py:75 (eager vs
graph check), adapter.py (model adapter ABC; here the model's ``forward``/``forward_sp`` is the adapter).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..models.transformer import AttnMeta, Transformer
from .kv_cache import PagedKVCache


def generate_buckets(max_bucket: int, num_buckets: int, multiple: int = 1) -> List[int]:
    """Roughly geometric bucket sizes ending at ``max_bucket``, each a multiple of ``multiple``."""
    if max_bucket <= 0:
        return []
    out = set()
    b = float(max(1, multiple))
    ratio = (max_bucket / b) ** (1.0 / max(1, num_buckets - 1)) if max_bucket > b else 1.0
    for _ in range(num_buckets):
        v = int(-(-int(round(b)) // multiple) * multiple)
        out.add(min(max(v, multiple), max_bucket))
        b *= max(ratio, 1.0001)
    out.add(-(-max_bucket // multiple) * multiple if max_bucket % multiple else max_bucket)
    return sorted(out)


class BatchSizeBucketing:
    def __init__(self, buckets: Seq[int]):
        self.buckets = sorted(set(buckets))

    def bucket_for(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        raise DecodeWidthExceedsGraphBucketError(f"decode width {n} exceeds the largest graph bucket "
                                                 f"{self.buckets[-1] if self.buckets else 0}")


class DecodeWidthExceedsGraphBucketError(RuntimeError):
    pass


@dataclass
class CaptureLedger:
    """Bytes of device memory each captured bucket added (the reference keeps the same ledger to size
    the KV pool after capture)."""
    per_bucket: Dict[int, int] = field(default_factory=dict)

    @property
    def total(self) -> int:
        return sum(self.per_bucket.values())


class DecodeGraphRunner:
    def __init__(self, model: Transformer, kv: PagedKVCache, max_batch: int, max_pages_per_seq: int,
                 num_buckets: int = 16, max_bucket: Optional[int] = None, sequence_parallel: bool = False):
        self.model, self.kv = model, kv
        self.dev = model.device
        self.sp = sequence_parallel
        self.world = model.comm.world if (model.comm is not None) else 1
        mult = self.world if self.sp else 1
        top = min(max_batch, max_bucket or max_batch)
        top = -(-top // mult) * mult
        self.bucketing = BatchSizeBucketing(generate_buckets(top, num_buckets, mult))
        self.max_pages = max_pages_per_seq
        B = top
        d = self.dev
        self.ids = torch.zeros(B, dtype=torch.int32, device=d)
        self.pos = torch.zeros(B, dtype=torch.int32, device=d)
        self.slots = torch.full((B,), -1, dtype=torch.int64, device=d)
        self.lens = torch.zeros(B, dtype=torch.int32, device=d)
        self.bt = torch.zeros(B, max_pages_per_seq, dtype=torch.int32, device=d)
        self.num_valid = torch.zeros(1, dtype=torch.int32, device=d)
        # state slot of each row (KDA recurrent state, or DeepSeek-V4 window / compressor state); -1 = padding row: it
        # is skipped or lands in a scratch slot, so warm-up and capture touch no sequence's state
        self.state_slots = (torch.full((B,), -1, dtype=torch.int32, device=d)
                            if (model.cfg.has_kda or model.cfg.is_v4) else None)
        pin = torch.cuda.is_available()
        self.h_state = torch.full((B,), -1, dtype=torch.int32, pin_memory=pin)
        self.h_ids = torch.zeros(B, dtype=torch.int32, pin_memory=pin)
        self.h_pos = torch.zeros(B, dtype=torch.int32, pin_memory=pin)
        self.h_slots = torch.full((B,), -1, dtype=torch.int64, pin_memory=pin)
        self.h_lens = torch.zeros(B, dtype=torch.int32, pin_memory=pin)
        self.h_bt = torch.zeros(B, max_pages_per_seq, dtype=torch.int32, pin_memory=pin)
        self.h_nv = torch.zeros(1, dtype=torch.int32, pin_memory=pin)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.outputs: Dict[int, torch.Tensor] = {}
        self.pool = None
        self.ledger = CaptureLedger()
        self.replays = 0
        self.h2d_bytes_per_step = 0
        # sampled tokens of the last step (device) and the deferred host read-back ring (2 pinned slots)
        self.tokens = torch.zeros(B, dtype=torch.int32, device=d)
        self._tok_local = torch.zeros(max(1, B // mult), dtype=torch.int32, device=d)
        self._ring = [torch.zeros(B, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._ring_ev = [torch.cuda.Event() if pin else None for _ in range(2)]
        self._ring_n = [0, 0]
        self._stage_ev = torch.cuda.Event() if pin else None
        self._ring_next = 0
        self._row_key = None
        self._scratch_reserved = False
        self._bt_keys: list = []                 # per staged row: key of the page list in the pinned block table

    # ------------------------------------------------------------------ capture
    def _meta(self, b: int) -> AttnMeta:
        return AttnMeta(mode="decode", positions=self.pos[:b], slot_mapping=self.slots[:b], block_table=self.bt[:b],
                        seqlens=self.lens[:b], num_valid=self.num_valid,
                        state_slots=None if self.state_slots is None else self.state_slots[:b])

    def _forward(self, b: int) -> torch.Tensor:
        if self.sp:
            return self.model.forward_sp(self.ids[:b], self._meta(b), self.kv)
        return self.model.forward(self.ids[:b], self._meta(b), self.kv)

    def capture(self, bucket: int) -> None:
        if bucket in self.graphs:
            return
        self.reserve_attention_scratch()
        free0 = torch.cuda.mem_get_info(self.dev)[0]
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            staged = None
            if self.state_slots is not None:         # recurrent state is not idempotent: warm up on no slot at all
                staged = self.state_slots.clone()
                self.state_slots.fill_(-1)
            for _ in range(2):                       # warm-up: caches, attributes, work lists
                self._forward(bucket)
            if staged is not None:
                self.state_slots.copy_(staged)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g, pool=self.pool):
            out = self._forward(bucket)
        torch.cuda.synchronize(self.dev)
        self.graphs[bucket] = g
        self.outputs[bucket] = out
        if self.world > 1:
            # ranks capture at different speeds; nobody replays (and waits on peers inside kernels) before
            # every rank holds the graph
            import torch.distributed as dist
            dist.barrier()
        self.ledger.per_bucket[bucket] = max(0, free0 - torch.cuda.mem_get_info(self.dev)[0])

    def reserve_attention_scratch(self) -> int:
        """Size the split-KV scratch of the MLA decode kernel for every bucket before anything is captured: the slot
        count (rows x head groups x splits) is not monotone in the batch size, and a captured launch keeps the
        addresses it was given.  Returns the largest slot count (0 when the model has no such kernel)."""
        cfg = self.model.cfg
        if not cfg.is_mla or cfg.is_v4 or torch.device(self.dev).type != "cuda" or self._scratch_reserved:
            return 0
        from ..ops import _ext, mla_kernel
        W = self.model.layout.tp_size
        sms = _ext.num_sms(self.dev)
        need = 0
        for b in self.bucketing.buckets:
            if self.model.attn_request_parallel and W > 1 and b % W == 0 and not cfg.has_dsa:
                rows, heads = b // W, cfg.num_heads            # own rows, every head
            else:
                rows, heads = b, cfg.num_heads // W
            tiles = [self.max_pages * self.kv.page_size // mla_kernel.KV_TILE]
            if cfg.has_dsa:                                    # sparse decode runs the same kernel over top-k rows
                tiles.append(-(-cfg.index_topk // mla_kernel.KV_TILE))
            for t in tiles:
                need = max(need, mla_kernel.reserve_decode_scratch(self.dev, [rows], heads, t, sms))
        self._scratch_reserved = True
        return need

    def capture_all(self) -> None:
        self.reserve_attention_scratch()
        for b in sorted(self.bucketing.buckets, reverse=True):   # largest first: smaller ones reuse its pool
            self.capture(b)

    # ------------------------------------------------------------------ replay
    def stage(self, ids: Optional[Seq[int]], pos: Seq[int], slots: Seq[int], lens: Seq[int], page_lists: Seq[Seq[int]],
              state_slots: Optional[Seq[int]] = None, page_keys: Optional[Seq] = None) -> int:
        """Fill the pinned staging buffers and enqueue the host->device copies.  Returns the bucket.
        ``page_keys[i]`` (optional) identifies the page list of row i, e.g. (sequence id, page count): rows whose
        key equals the one staged last time keep their block-table row, and when no row changed the block table is
        not copied at all (page lists change only at page boundaries)."""
        n = len(pos)
        b = self.bucketing.bucket_for(n)
        if self._stage_ev is not None:
            self._stage_ev.synchronize()            # the copies of the step staged before have left the pinned buffers
        if self.state_slots is not None:
            self.h_state[:b] = -1
            if state_slots is not None:
                self.h_state[:n] = torch.as_tensor(state_slots, dtype=torch.int32)
            self.state_slots[:b].copy_(self.h_state[:b], non_blocking=True)
        if ids is not None:
            self.h_ids[:n] = torch.as_tensor(ids, dtype=torch.int32)
        self.h_pos[:n] = torch.as_tensor(pos, dtype=torch.int32)
        self.h_slots[:n] = torch.as_tensor(slots, dtype=torch.int64)
        self.h_lens[:n] = torch.as_tensor(lens, dtype=torch.int32)
        if b > n:
            self.h_ids[n:b] = 0
            self.h_pos[n:b] = 0
            self.h_slots[n:b] = -1
            self.h_lens[n:b] = 0
        bt_rows = 0
        for i, pl in enumerate(page_lists):
            if page_keys is not None:
                if i < len(self._bt_keys) and self._bt_keys[i] == page_keys[i]:
                    continue
                if i < len(self._bt_keys):
                    self._bt_keys[i] = page_keys[i]
                else:
                    self._bt_keys.append(page_keys[i])
            k = len(pl)
            if k > self.max_pages:
                raise ValueError(f"row {i} holds {k} pages but the captured block table has {self.max_pages} columns "
                                 f"(max_pages_per_seq)")
            self.h_bt[i, :k] = torch.as_tensor(pl, dtype=torch.int32)
            bt_rows += 1
        if page_keys is None:
            self._bt_keys = []
        else:
            del self._bt_keys[n:]
        self.h_nv[0] = n
        nb = True
        if ids is not None:
            self.ids[:b].copy_(self.h_ids[:b], non_blocking=nb)
        else:                                        # feed the tokens sampled by the previous step (device side)
            self.ids[:n].copy_(self.tokens[:n], non_blocking=nb)
        self.pos[:b].copy_(self.h_pos[:b], non_blocking=nb)
        self.slots[:b].copy_(self.h_slots[:b], non_blocking=nb)
        self.lens[:b].copy_(self.h_lens[:b], non_blocking=nb)
        if bt_rows:
            self.bt[:n].copy_(self.h_bt[:n], non_blocking=nb)
        self.num_valid.copy_(self.h_nv, non_blocking=nb)
        if self._stage_ev is not None:
            self._stage_ev.record()
        self.h2d_bytes_per_step = (b * (4 + 8 + 4) + (b * 4 if ids is not None else 0)
                                   + (n * self.max_pages * 4 if bt_rows else 0) + 4)
        return b

    def replay(self, bucket: int, n: int) -> torch.Tensor:
        if bucket not in self.graphs:
            self.capture(bucket)
        self.graphs[bucket].replay()
        self.replays += 1
        out = self.outputs[bucket]
        if self.sp:
            return out                              # own rows of the bucket; caller slices by rank
        return out[:n]

    # ------------------------------------------------------------------ deferred token read-back
    def decode_async(self, pos: Seq[int], slots: Seq[int], lens: Seq[int], page_lists: Seq[Seq[int]],
                     ids: Optional[Seq[int]] = None, sampler=None) -> int:
        """One full decode step without a host synchronisation: stage inputs (host -> device), replay the
        graph, sample on the device, start the device -> host copy of the tokens into a pinned ring slot.
        ``ids is None`` feeds the tokens sampled by the previous step.  Returns a handle for ``read``.
        The host sees a step's tokens one step late (the reference defers its token read-back the same
        way: batchgen/worker/deferred_readback.py:57)."""
        from ..ops import sampling as sampling_ops
        n = len(pos)
        b = self.stage(ids, pos, slots, lens, page_lists)
        logits = self.replay(b, n)
        if self.sp:
            import torch.distributed as dist
            tl = self._tok_local[: b // self.world]
            (sampler or sampling_ops.greedy)(logits, tl)
            dist.all_gather_into_tensor(self.tokens[:b], tl)
        else:
            (sampler or sampling_ops.greedy)(logits, self.tokens[:n])
        return self.start_readback(n)

    def start_readback(self, n: int) -> int:
        """Start the device -> host copy of the first ``n`` sampled tokens into the next pinned ring slot."""
        slot = self._ring_next
        self._ring_next ^= 1
        self._ring[slot][:n].copy_(self.tokens[:n], non_blocking=True)
        if self._ring_ev[slot] is not None:
            self._ring_ev[slot].record()
        self._ring_n[slot] = n
        return slot

    def read(self, handle: int) -> torch.Tensor:
        """Tokens of the step that returned ``handle`` (blocks until its copy has landed)."""
        if self._ring_ev[handle] is not None:
            self._ring_ev[handle].synchronize()
        return self._ring[handle][: self._ring_n[handle]]

    def decode(self, engine, rows, ids, pos, slots, lens):
        """Engine hook (``Engine.graph_runner``): (logits, bucket) of the step.  ``None`` entries of ``rows`` are empty
        rows that pad a rank's block in request-split decode; their logits are returned too and ignored by the
        engine.  Without sequence parallelism the logits cover ``rows``; with it they cover this rank's block of the
        bucket (rows past ``len(rows)`` are padding)."""
        b = self.stage(ids, pos, slots, lens, [s.gpu_pages if s is not None else [] for s in rows],
                       [s.state_slot if s is not None else -1 for s in rows] if self.state_slots is not None else None,
                       page_keys=[(s.global_idx, len(s.gpu_pages), sum(s.gpu_pages)) if s is not None else (-1, 0, 0)
                                  for s in rows])
        key = tuple(id(s) for s in rows)
        if key != self._row_key and self.model.cfg.is_mla and torch.device(self.dev).type == "cuda":
            # batch membership changed: put the longest sequences first in the attention work lists
            from ..ops import mla_kernel
            self._row_key = key
            padded = list(lens) + [0] * (b - len(lens))
            W = self.model.layout.tp_size
            if self.model.attn_request_parallel and W > 1 and b % W == 0:
                r = self.model.layout.tp_rank            # request-split core: this rank attends over its own block
                padded = padded[r * (b // W):(r + 1) * (b // W)]
            mla_kernel.reorder_decode_work(self.dev, padded)
        return self.replay(b, len(rows)), b


def compare_eager_vs_graph(runner: DecodeGraphRunner, ids, pos, slots, lens, page_lists, atol=0.0, rtol=0.0):
    """Run one staged step eagerly and through the graph; returns (max_abs_diff, equal_bits).  The eager
    run comes second so that the KV rows written by both are identical."""
    b = runner.stage(ids, pos, slots, lens, page_lists)
    n = len(ids)
    g = runner.replay(b, n).clone()
    torch.cuda.synchronize(runner.dev)
    e = runner._forward(b)
    e = e if runner.sp else e[:n]
    torch.cuda.synchronize(runner.dev)
    diff = (g.float() - e.float()).abs().max().item()
    return diff, bool(torch.equal(g, e))
