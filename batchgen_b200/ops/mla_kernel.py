"""Host side of the tcgen05 paged-MLA kernel: work lists, split-KV scratch and launches.

A *work item* is one CTA: up to ``NCOL`` (query, head) columns of one sequence over a contiguous range
of KV tiles.  Decode work lists depend only on (batch, heads, splits) — sequence lengths are read on
the device — so they are built once, cached on the device and are safe to replay in a CUDA graph.
Prefill work lists are built per micro-batch from the host-side ``cu_seqlens``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Sequence, Tuple

import torch

from . import _ext

KV_TILE = 64
_DECODE_WORK: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor, int]] = {}
_SCRATCH: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def _geometry(H: int, prefill: bool) -> Tuple[int, int]:
    """(heads_per_group, ncol)."""
    if H % 64 == 0:
        return 64, 64
    if H % 32 == 0:
        return 32, (64 if prefill else 32)
    if H % 16 == 0:
        return 16, (32 if prefill else 16)
    if H % 8 == 0:
        return 8, (32 if prefill else 16)
    raise ValueError(f"the MLA kernel needs a multiple of 8 heads per rank, got {H}")


_RETIRED: list = []      # replaced scratch buffers: a captured CUDA graph may still hold their addresses


def _scratch(device, slots: int, ncol: int):
    """Split-KV partial buffers for ``slots`` work items.  A launch captured in a CUDA graph keeps the addresses it
    was given, so a buffer that is outgrown is never freed: it moves to ``_RETIRED`` and the graphs that captured it
    keep working on it.  ``reserve_decode_scratch`` sizes the buffer for every bucket up front, so that growth after
    the first capture does not happen at all in the graph runner."""
    key = (str(device), ncol)
    cur = _SCRATCH.get(key)
    if cur is None or cur[0].shape[0] < slots:
        if cur is not None:
            _RETIRED.append(cur)
        n = max(slots, 256)
        cur = (torch.empty(n, ncol, 512, dtype=torch.float32, device=device),
               torch.empty(n, ncol, 2, dtype=torch.float32, device=device))
        _SCRATCH[key] = cur
    return cur


def decode_splits(B: int, H: int, max_tiles: int, sms: int) -> int:
    """Split count of a decode launch.  A CTA costs about 12 us before and after its tiles (query load, TMEM,
    pipeline fill, partial store), a 64-token tile 1.7 - 2.7 us: about two rounds of CTAs over the SMs balance
    ragged lengths (longest first, see reorder_decode_work) without paying that fixed cost too often.  Measured on
    48 rows x 16 heads x 4096 tokens with 13 splits (four rounds): 87 us, 0.41 of copy bandwidth."""
    hpg, _ = _geometry(H, prefill=False)
    ctas = B * (H // hpg)
    return max(1, min(16, int(2.0 * sms / ctas + 0.5), max(1, max_tiles) // 4))


def decode_slots(B: int, H: int, max_tiles: int, sms: int) -> int:
    """Work items (= scratch slots) of a decode launch of batch ``B``; not monotone in ``B``."""
    hpg, _ = _geometry(H, prefill=False)
    return B * (H // hpg) * decode_splits(B, H, max_tiles, sms)


def reserve_decode_scratch(device, batch_sizes: Sequence[int], H: int, max_tiles: int, sms: int) -> int:
    """Size the split-KV scratch once for the largest slot count over ``batch_sizes`` (the graph buckets), before the
    first capture.  Returns that slot count."""
    _, ncol = _geometry(H, prefill=False)
    need = max(decode_slots(b, H, max_tiles, sms) for b in batch_sizes)
    _scratch(device, need, ncol)
    return need


def _qpe_view(q_pe: torch.Tensor):
    R, H, D = q_pe.shape
    if q_pe.stride(2) != 1 or q_pe.stride(0) != H * q_pe.stride(1) or (q_pe.stride(1) * 2) % 16 != 0 \
            or q_pe.data_ptr() % 16 != 0:
        q_pe = q_pe.contiguous()
    return q_pe, q_pe.stride(1)


def _launch(q_abs, q_pe, cache, work, n_work, block_table, seqlens, out, part_o, part_ml, H, hpg, ncol, scale):
    q_pe, qpe_stride = _qpe_view(q_pe)
    q_abs, qabs_stride = _qpe_view(q_abs)          # same rule: unit inner stride, dense over heads, 16-byte steps
    R = q_abs.shape[0]
    P, S, D = cache.shape
    rc = _ext.lib().bg_mla_attention_strided(
        _ext.ptr(q_abs), ctypes.c_longlong(qabs_stride), _ext.ptr(q_pe), ctypes.c_longlong(qpe_stride),
        ctypes.c_longlong(R * H), _ext.ptr(cache),
        ctypes.c_longlong(P * S), _ext.ptr(work), ctypes.c_int(n_work), _ext.ptr(block_table),
        ctypes.c_int(block_table.stride(0)), _ext.ptr(seqlens), _ext.ptr(out), _ext.ptr(part_o), _ext.ptr(part_ml),
        ctypes.c_int(H), ctypes.c_int(hpg), ctypes.c_int(ncol), ctypes.c_float(scale),
        _ext.ptr(_ext.status_word(q_abs.device)), _ext.stream())
    _ext.check(rc, "bg_mla_attention")


def _decode_work_lists(order: Sequence[int], groups: int, num_splits: int):
    """Work items (one CTA each) and merge items for decode rows taken in ``order``."""
    B = len(order)
    rows = torch.as_tensor(list(order), dtype=torch.int32)
    b = rows.repeat_interleave(groups * num_splits)
    g = torch.arange(groups, dtype=torch.int32).repeat_interleave(num_splits).repeat(B)
    sp = torch.arange(num_splits, dtype=torch.int32).repeat(B * groups)
    w = torch.zeros(B * groups * num_splits, 8, dtype=torch.int32)
    w[:, 0] = b; w[:, 1] = 1; w[:, 2] = b; w[:, 3] = -1; w[:, 4] = sp; w[:, 5] = num_splits; w[:, 6] = g
    w[:, 7] = torch.arange(w.shape[0], dtype=torch.int32)
    items = torch.zeros(B * groups, 5, dtype=torch.int32)
    items[:, 0] = rows.repeat_interleave(groups); items[:, 1] = 1
    items[:, 2] = torch.arange(groups, dtype=torch.int32).repeat(B)
    items[:, 3] = torch.arange(B * groups, dtype=torch.int32) * num_splits; items[:, 4] = num_splits
    return w, items


def reorder_decode_work(device, lengths: Sequence[int]) -> int:
    """Rewrite, in place, every cached decode work list of batch size ``len(lengths)`` on ``device`` so that
    the longest sequences come first (longest-processing-time order for the hardware CTA scheduler).  The
    lists are static device buffers, so CUDA graphs that captured a decode launch pick the new order up on
    their next replay.  Any order is correct; a stale one only balances worse.  Returns lists rewritten."""
    B = len(lengths)
    order = sorted(range(B), key=lambda i: -int(lengths[i]))
    n = 0
    for (dev, b, H, splits), (w_d, items_d, _) in _DECODE_WORK.items():
        if dev != str(device) or b != B:
            continue
        groups = items_d.shape[0] // B
        w, items = _decode_work_lists(order, groups, splits)
        w_d.copy_(w, non_blocking=False)
        items_d.copy_(items, non_blocking=False)
        n += 1
    return n


_PERSIST: Dict[str, Tuple[torch.Tensor, ...]] = {}
MAX_PERSIST_PAIRS = 2048
PERSIST = os.environ.get("BG_MLA_PERSIST", "1") != "0"


def _persist_scratch(dev):
    """Fixed-size scratch of the persistent decode kernel (partials of cut pairs, per-pair arrival counters, every
    CTA's copy of the tile prefix sums).  Sized by the SM count alone, allocated once per device and never replaced,
    so launches captured in CUDA graphs keep valid addresses."""
    key = str(dev)
    cur = _PERSIST.get(key)
    if cur is None:
        ctas = _ext.num_sms(dev)
        cur = (torch.empty(2 * ctas * 64 * 512, dtype=torch.float32, device=dev),
               torch.empty(2 * ctas * 64 * 2, dtype=torch.float32, device=dev),
               torch.zeros(MAX_PERSIST_PAIRS * 16, dtype=torch.int32, device=dev),      # one counter per (sequence, group)
               torch.empty(ctas * (MAX_PERSIST_PAIRS + 1), dtype=torch.int32, device=dev))
        _PERSIST[key] = cur
    return cur


def mla_decode_persist(q_abs, q_pe, cache, block_table, seqlens, scale):
    """Persistent decode kernel (``csrc/mla_decode_persist.cu``): heads % 64 == 0, one query per sequence.  The KV
    tiles of the whole batch are cut into equal shares per SM on the device, from the device-side lengths."""
    B, H, _ = q_abs.shape
    dev = q_abs.device
    q_pe, qpe_stride = _qpe_view(q_pe)
    q_abs, qabs_stride = _qpe_view(q_abs)
    P, S, D = cache.shape
    part_o, part_ml, counters, prefix = _persist_scratch(dev)
    out = torch.empty(B, H, 512, dtype=torch.bfloat16, device=dev)
    rc = _ext.lib().bg_mla_decode_persist(
        _ext.ptr(q_abs), ctypes.c_longlong(qabs_stride), _ext.ptr(q_pe), ctypes.c_longlong(qpe_stride), ctypes.c_int(B),
        ctypes.c_int(H), _ext.ptr(cache), ctypes.c_longlong(P * S), _ext.ptr(block_table),
        ctypes.c_int(block_table.stride(0)), _ext.ptr(seqlens), _ext.ptr(out), _ext.ptr(part_o), _ext.ptr(part_ml),
        _ext.ptr(counters), _ext.ptr(prefix), ctypes.c_int(_ext.num_sms(dev)), ctypes.c_float(scale),
        _ext.ptr(_ext.status_word(dev)), _ext.stream())
    _ext.check(rc, "bg_mla_decode_persist")
    return out


def mla_decode_tc(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora, num_splits: int = 0):
    """q_abs [B, H, 512], q_pe [B, H, 64] -> [B, H, 512]."""
    B, H, _ = q_abs.shape
    dev = q_abs.device
    if PERSIST and num_splits <= 0 and H % 64 == 0 and B <= MAX_PERSIST_PAIRS and H // 64 <= 16:
        return mla_decode_persist(q_abs, q_pe, cache, block_table, seqlens, scale)
    # q_abs may be a strided view (see _launch); only a non-unit inner stride forces a copy there
    hpg, ncol = _geometry(H, prefill=False)
    groups = H // hpg
    if num_splits <= 0:
        num_splits = decode_splits(B, H, (block_table.shape[1] * cache.shape[1]) // KV_TILE, _ext.num_sms(dev))
    key = (str(dev), B, H, num_splits)
    cached = _DECODE_WORK.get(key)
    if cached is None:
        w, items = _decode_work_lists(list(range(B)), groups, num_splits)
        cached = (w.to(dev), items.to(dev), w.shape[0])
        _DECODE_WORK[key] = cached
    work, items, n_work = cached
    out = torch.empty(B, H, 512, dtype=torch.bfloat16, device=dev)
    part_o = part_ml = None
    if num_splits > 1:
        part_o, part_ml = _scratch(dev, n_work, ncol)
    _launch(q_abs, q_pe, cache, work, n_work, block_table, seqlens, out, part_o, part_ml, H, hpg, ncol, scale)
    if num_splits > 1:
        rc = _ext.lib().bg_mla_merge(_ext.ptr(part_o), _ext.ptr(part_ml), _ext.ptr(items), ctypes.c_int(items.shape[0]),
                                     _ext.ptr(out), ctypes.c_int(ncol), ctypes.c_int(H), ctypes.c_int(hpg),
                                     _ext.stream())
        _ext.check(rc, "bg_mla_merge")
    return out


def mla_prefill_tc(q_abs, q_pe, cache, block_table, cu_seqlens: Sequence[int], ctx_lens: Sequence[int], scale,
                   kv_lora):
    """Varlen causal MLA: query j of sequence i attends to cache positions 0 .. ctx_i + j."""
    T, H, _ = q_abs.shape
    dev = q_abs.device
    # (strided q_abs views are accepted, see _launch)
    hpg, ncol = _geometry(H, prefill=True)
    groups, qt = H // hpg, ncol // hpg
    rows = []
    for i in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        if b <= a:
            continue
        q0 = torch.arange(a, b, qt)
        n_q = torch.clamp(torch.tensor(b) - q0, max=qt)
        w = torch.zeros(q0.numel(), 8, dtype=torch.int32)
        w[:, 0] = q0; w[:, 1] = n_q; w[:, 2] = i; w[:, 3] = int(ctx_lens[i]) + (q0 - a); w[:, 4] = 0; w[:, 5] = 1
        rows.append(w)
    out = torch.empty(T, H, 512, dtype=torch.bfloat16, device=dev)
    if not rows:
        return out
    w = torch.cat(rows, 0)
    w = w[torch.argsort(w[:, 3], descending=True)]                 # longest KV ranges first
    w = w.repeat_interleave(groups, 0)
    w[:, 6] = torch.arange(groups, dtype=torch.int32).repeat(w.shape[0] // groups)
    work = w.contiguous().to(dev)
    dummy_len = torch.zeros(1, dtype=torch.int32, device=dev)
    _launch(q_abs, q_pe, cache, work, work.shape[0], block_table, dummy_len, out, None, None, H, hpg, ncol, scale)
    return out
