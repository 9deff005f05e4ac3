"""Paged KV storage: device pool, host (CPU-DRAM) tier, page allocators and movers.

Device pool: one tensor ``[layers, pages, page_size, row]`` (row = 576 for MLA latent), plus, for
DSA models, a second region of FP8 index keys ``[idx_layers, pages, page_size, 128]`` with fp32
scales — the same logical page id addresses both regions (the reference's "dual" coordinators,
batchgen/kv_cache/dual_kv_cache_coordinator.py).  Host tier: the same layout in pinned memory.
Pages are reference counted so that sequences sharing a prefix share physical pages
(batchgen/worker/decode.py:169-199: one physical page per distinct host page).

Reference parity: batchgen/kv_cache/gpu_paged_kv_manager.py:110-761 (pool ``[layers, pages, 64,
heads, dim]``, page-table state), core/KV_Storage/host_paged_kv_* (host pages, async load/offload).
The native host-tier backend lives in ``core/csrc``; this module is its Python front.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence as Seq, Tuple

import torch

from ..config import ModelConfig

FP8 = torch.float8_e4m3fn


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    """Free-list allocator with reference counts."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._ref = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._ref[p] = 1
        return out

    def share(self, pages: Seq[int]) -> None:
        for p in pages:
            assert self._ref[p] > 0, f"page {p} is not live"
            self._ref[p] += 1

    def free(self, pages: Seq[int]) -> None:
        for p in pages:
            assert self._ref[p] > 0, f"double free of page {p}"
            self._ref[p] -= 1
            if self._ref[p] == 0:
                self._free.append(p)

    def refcount(self, page: int) -> int:
        return self._ref[page]


def host_page_bytes(cfg: ModelConfig, page_size: int, kv_elem_bytes: int = 2) -> int:
    """Bytes of one page over all layers (latent KV, then DSA index keys and their scales): the page size of the
    node-shared host region, which the server computes without building a model."""
    if cfg.is_v4:
        return sum(v4_entries_per_page(r, page_size) * (cfg.head_dim + (cfg.index_head_dim if r == 4 else 0))
                   for r in cfg.compress_ratios if r) * kv_elem_bytes
    kv_layers = sum(1 for l in range(cfg.num_layers) if not cfg.layer_is_kda(l))
    b = kv_layers * page_size * cfg.kv_cache_dim * kv_elem_bytes
    if cfg.has_dsa:
        n = len(list(cfg.indexer_full_layers) or range(cfg.num_layers))
        b += n * page_size * (cfg.index_head_dim + 4)
    return b


def v4_entries_per_page(ratio: int, page_size: int) -> int:
    """Pooled entries a page of ``page_size`` tokens holds at compression ``ratio``.  Entry c (tokens c*ratio ..)
    lives in the page of its first token, at slot ((c * ratio) % page_size) // ratio; when the ratio exceeds the
    page only every (ratio / page_size)-th page of a sequence carries an entry."""
    if ratio <= page_size:
        assert page_size % ratio == 0, (ratio, page_size)
        return page_size // ratio
    assert ratio % page_size == 0, (ratio, page_size)
    return 1


class PagedKVCache:
    """One tier (device or pinned host) of paged KV."""

    def __init__(self, cfg: ModelConfig, num_pages: int, page_size: int, device, dtype: torch.dtype,
                 pinned: bool = False, row_dim: Optional[int] = None, state_slots: int = 0,
                 state_heads: Optional[int] = None):
        self.cfg, self.num_pages, self.page_size = cfg, num_pages, page_size
        self.device = torch.device(device)
        self.row_dim = row_dim or cfg.kv_cache_dim
        pin = pinned and self.device.type == "cpu" and torch.cuda.is_available()
        # KDA layers keep no paged KV: layer l's rows live at index kv_index[l] of the pool
        kv_layers = [] if cfg.is_v4 else [l for l in range(cfg.num_layers) if not cfg.layer_is_kda(l)]
        self.kv_index = {l: i for i, l in enumerate(kv_layers)}
        self.kv = torch.zeros(len(kv_layers), num_pages, page_size, self.row_dim, dtype=dtype, device=self.device,
                              pin_memory=pin)
        self.idx_layers: Dict[int, int] = {}
        self.idx_k = self.idx_s = None
        if cfg.has_dsa:
            layers = list(cfg.indexer_full_layers) or list(range(cfg.num_layers))
            self.idx_layers = {l: i for i, l in enumerate(layers)}
            self.idx_k = torch.zeros(len(layers), num_pages, page_size, cfg.index_head_dim, dtype=FP8,
                                     device=self.device, pin_memory=pin)
            self.idx_s = torch.zeros(len(layers), num_pages, page_size, dtype=torch.float32, device=self.device,
                                     pin_memory=pin)
        # DeepSeek-V4: pooled KV entries (and the indexer's pooled keys on ratio-4 layers) are the only paged rows;
        # layer l's pool is [pages, entries per page, width]
        self.v4_comp: Dict[int, torch.Tensor] = {}
        self.v4_idx: Dict[int, torch.Tensor] = {}
        for l, r in enumerate(cfg.compress_ratios):
            if r:
                epp = v4_entries_per_page(r, page_size)
                # one page more than the allocator hands out: rows without a sequence (padding) write there
                self.v4_comp[l] = torch.zeros(num_pages + 1, epp, cfg.head_dim, dtype=dtype, device=self.device, pin_memory=pin)
                if r == 4:
                    self.v4_idx[l] = torch.zeros(num_pages + 1, epp, cfg.index_head_dim, dtype=dtype, device=self.device,
                                                 pin_memory=pin)
        self.alloc = PageAllocator(num_pages)
        # per-sequence state (device tier only): recurrent state of the KDA layers, or the window rings and
        # compressor windows of a DeepSeek-V4 model
        self.state = None
        if cfg.has_kda and state_slots:
            self.state = StateSlotPool(cfg, state_slots, self.device, state_heads)
        elif cfg.is_v4 and state_slots:
            self.state = V4StatePool(cfg, state_slots, self.device)

    # ---- views used by the model
    def latent(self, layer: int) -> torch.Tensor:
        return self.kv[self.kv_index[layer]]

    def index_keys(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        i = self.idx_layers[layer]
        return self.idx_k[i], self.idx_s[i]

    def write_index_keys(self, layer: int, kq: torch.Tensor, ks: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        i = self.idx_layers[layer]
        valid = slot_mapping >= 0
        slots = slot_mapping[valid].long()
        self.idx_k[i].view(-1, self.cfg.index_head_dim).view(torch.uint8)[slots] = kq[valid].view(torch.uint8)
        self.idx_s[i].view(-1)[slots] = ks[valid]

    def _v4_pools(self) -> List[torch.Tensor]:
        return list(self.v4_comp.values()) + list(self.v4_idx.values())

    def bytes_per_page(self) -> int:
        if self.cfg.is_v4:
            return sum(t[0].numel() * t.element_size() for t in self._v4_pools())
        b = self.kv[0, 0].numel() * self.kv.element_size() * self.kv.shape[0]
        if self.idx_k is not None:
            b += len(self.idx_layers) * (self.idx_k[0, 0].numel() + 4 * self.page_size)
        return b

    # ---- page movement between tiers
    def copy_pages_from(self, other: "PagedKVCache", src_pages: Seq[int], dst_pages: Seq[int],
                        stream: Optional["torch.cuda.Stream"] = None) -> None:
        """self[:, dst] <- other[:, src] for every layer (both regions)."""
        if not src_pages:
            return
        src = torch.as_tensor(list(src_pages), dtype=torch.long)
        dst = torch.as_tensor(list(dst_pages), dtype=torch.long)
        ctx = torch.cuda.stream(stream) if stream is not None else _NullCtx()
        with ctx:
            if self.cfg.is_v4:
                for mine, theirs in zip(self._v4_pools(), other._v4_pools()):
                    if self.device.type == other.device.type == "cpu":
                        mine[dst] = theirs[src]
                    else:
                        for s_, d_ in zip(src.tolist(), dst.tolist()):
                            mine[d_].copy_(theirs[s_], non_blocking=True)
                return
            if self.device.type == other.device.type == "cpu":
                self.kv[:, dst] = other.kv[:, src]
                if self.idx_k is not None:
                    self.idx_k.view(torch.uint8)[:, dst] = other.idx_k.view(torch.uint8)[:, src]
                    self.idx_s[:, dst] = other.idx_s[:, src]
                return
            for s, d in zip(src.tolist(), dst.tolist()):
                self.kv[:, d].copy_(other.kv[:, s], non_blocking=True)
                if self.idx_k is not None:
                    self.idx_k[:, d].copy_(other.idx_k[:, s], non_blocking=True)
                    self.idx_s[:, d].copy_(other.idx_s[:, s], non_blocking=True)


class StateSlotPool:
    """Per-sequence recurrent state of the KDA layers: ``rec[i]`` [slots, H, D, D] fp32 and ``conv[i]``
    [slots, 3 H D, 3] fp32 for the i-th KDA layer, plus a free list of slots.  A sequence holds one slot from
    its first prefill chunk until it completes or is evicted (its state cannot be rebuilt from paged KV).

    Reference parity: the KDA / compressed state GPU managers and their sequence-slot caps
    (batchgen/kv_cache/kda_state_gpu_manager.py, batchgen/prefill.py:374-387)."""

    def __init__(self, cfg: ModelConfig, num_slots: int, device, heads: Optional[int] = None):
        self.layers = {l: i for i, l in enumerate(cfg.kda_layers)}
        H, D = heads or cfg.kda_num_heads, cfg.kda_head_dim
        self.num_slots = num_slots
        self.rec = torch.zeros(len(self.layers), num_slots, H, D, D, dtype=torch.float32, device=device)
        self.conv = torch.zeros(len(self.layers), num_slots, 3 * H * D, 3, dtype=torch.float32, device=device)
        self._free = list(range(num_slots - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        return self._free.pop()

    def release(self, slot: int) -> None:
        assert 0 <= slot < self.num_slots and slot not in self._free
        self._free.append(slot)

    def layer(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        i = self.layers[layer]
        return self.conv[i], self.rec[i]


class V4StatePool:
    """Per-sequence state of a DeepSeek-V4 model, one fp32 row per slot: for every layer the sliding-window ring of
    raw KV rows ([window, D], row = position % window), and on compressed layers the compressor's pending windows
    (projections and gate scores of the tokens not pooled yet; with overlapped windows also the previous window),
    twice on ratio-4 layers (attention entries and index keys).  ``rec`` / ``conv`` follow ``StateSlotPool`` so the
    host store parks a row the same way (``conv`` is an empty placeholder).

    Reference parity: the compressed-ratio GPU KV variant and its per-sequence compressor state
    (batchgen/kv_cache/gpu_paged_kv_manager.py, SWA / compressed-ratio variants)."""

    def __init__(self, cfg: ModelConfig, num_slots: int, device):
        self.cfg, self.num_slots = cfg, num_slots
        D, Di, win = cfg.head_dim, cfg.index_head_dim, cfg.sliding_window
        self.offsets: Dict[Tuple[int, str], Tuple[int, Tuple[int, ...]]] = {}
        n = 0
        for l, r in enumerate(cfg.compress_ratios):
            parts = [("ring", (win, D))]
            if r:
                c = 2 if r == 4 else 1
                parts += [("kv", (c * r, c * D)), ("score", (c * r, c * D))]
                if r == 4:
                    parts += [("idx_kv", (2 * r, 2 * Di)), ("idx_score", (2 * r, 2 * Di))]
            for name, shape in parts:
                self.offsets[(l, name)] = (n, shape)
                n += shape[0] * shape[1]
        assert n == cfg.v4_state_floats_per_seq()
        # row ``num_slots`` is scratch: decode rows without a sequence park their writes there
        self.rec = torch.zeros(1, num_slots + 1, n, dtype=torch.float32, device=device)
        self.conv = torch.zeros(1, num_slots + 1, 1, dtype=torch.float32, device=device)
        self._free = list(range(num_slots - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        return self._free.pop()

    def release(self, slot: int) -> None:
        assert 0 <= slot < self.num_slots and slot not in self._free
        self._free.append(slot)

    def view(self, slot: int, layer: int, name: str) -> torch.Tensor:
        """A writable view of one part of ``slot``'s state."""
        off, shape = self.offsets[(layer, name)]
        return self.rec[0, slot, off: off + shape[0] * shape[1]].view(shape)


class HostStateStore:
    """Host-memory store of recurrent (KDA) state items: a sequence that leaves the decode batch parks its state
    here (pinned memory, copies on the engine's copy stream) and gives its device slot to another sequence; the
    state returns to any free slot when the sequence is scheduled again.

    Reference parity: the compressed-state host manager with asynchronous offload / load of state items
    (core/KV_Storage/compressed_state_host_manager.h)."""

    def __init__(self, pool: StateSlotPool, num_items: int, pinned: bool = True):
        pin = pinned and torch.cuda.is_available()
        self.rec = torch.zeros(pool.rec.shape[0], num_items, *pool.rec.shape[2:], dtype=pool.rec.dtype, pin_memory=pin)
        self.conv = torch.zeros(pool.conv.shape[0], num_items, *pool.conv.shape[2:], dtype=pool.conv.dtype, pin_memory=pin)
        self.num_items = num_items
        self._free = list(range(num_items - 1, -1, -1))
        self.offloads = self.loads = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    def reserve(self) -> int:
        """Take a free item without filling it (a migrated row's state is received straight into it)."""
        if not self._free:
            raise OutOfPages("no free host state item")
        return self._free.pop()

    def offload(self, pool: StateSlotPool, slot: int, stream=None) -> int:
        """Copy the state of ``slot`` (all KDA layers) to a free item; returns the item.  The caller releases the
        slot once the copy stream has been synchronised or ordered before the slot's next writer."""
        item = self.reserve()
        ctx = torch.cuda.stream(stream) if stream is not None else _NullCtx()
        with ctx:
            self.rec[:, item].copy_(pool.rec[:, slot], non_blocking=True)
            self.conv[:, item].copy_(pool.conv[:, slot], non_blocking=True)
        self.offloads += 1
        return item

    def load(self, pool: StateSlotPool, item: int, slot: int, stream=None) -> None:
        ctx = torch.cuda.stream(stream) if stream is not None else _NullCtx()
        with ctx:
            pool.rec[:, slot].copy_(self.rec[:, item], non_blocking=True)
            pool.conv[:, slot].copy_(self.conv[:, item], non_blocking=True)
        self.loads += 1

    def release(self, item: int) -> None:
        assert 0 <= item < self.num_items and item not in self._free
        self._free.append(item)


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def slots_for_range(pages: Seq[int], start: int, end: int, page_size: int) -> List[int]:
    """Flat slot ids of token positions [start, end) of a sequence whose pages are ``pages``."""
    return [pages[p // page_size] * page_size + p % page_size for p in range(start, end)]


def build_block_table(page_lists: Seq[Seq[int]], device, min_width: int = 1) -> torch.Tensor:
    width = max(min_width, max((len(p) for p in page_lists), default=1))
    bt = torch.zeros(len(page_lists), width, dtype=torch.int32)
    for i, p in enumerate(page_lists):
        if p:
            bt[i, : len(p)] = torch.as_tensor(list(p), dtype=torch.int32)
    return bt.to(device)
