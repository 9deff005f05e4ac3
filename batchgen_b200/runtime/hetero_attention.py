"""Slot-based host KV with heterogeneous decode attention (the older, non-paged arrangement).

Every sequence owns one *slot* of host memory that holds its whole KV, layer by layer, for up to ``max_len`` tokens
(no pages, no block tables).  Decode attention over that storage runs in one of three modes:

* mode 0 (device): the layer's KV of the batch is copied into one of two device buffers while the other one is being
  read (layer l + 1 streams in while layer l computes), and attention runs on the device;
* mode 1 (host): attention runs on the host cores over the slot memory itself (AVX2 / OpenMP GQA kernel,
  ``core/csrc/cpu_attention.cpp``); only the query rows and the outputs cross the bus;
* mode 2 (split): the longest ``host_fraction`` of the rows run on the host, the rest on the device, concurrently.

The serving engine uses the paged tiers (``runtime/kv_cache.py``, ``runtime/host_tier.py``); this module is the
counterpart of the arrangement the reference keeps for its attention modes 0 - 2 and is not on the serving path.

Reference parity: core/KV_Storage/KV_Storage.{h,cpp} (slot-based host KV), core/GPU_KV_Buffer/ (double-buffered device
KV), core/Hetero_Attn/Hetero_Attn.{h,cpp} (orchestration of the modes over the CPU GQA kernel).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import ref


class SlotKVStorage:
    """Host KV in slots: ``k`` / ``v`` [layers, slots, max_len, Hkv, D] bf16 (pinned when a GPU is present)."""

    def __init__(self, layers: int, slots: int, max_len: int, num_kv_heads: int, head_dim: int, pinned: bool = True):
        pin = pinned and torch.cuda.is_available()
        shape = (layers, slots, max_len, num_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, pin_memory=pin)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, pin_memory=pin)
        self.layers, self.slots, self.max_len, self.hkv, self.d = layers, slots, max_len, num_kv_heads, head_dim
        self.lens = [0] * slots
        self._free = list(range(slots - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise MemoryError("no free KV slot")
        s = self._free.pop()
        self.lens[s] = 0
        return s

    def release(self, slot: int) -> None:
        assert 0 <= slot < self.slots and slot not in self._free
        self.lens[slot] = 0
        self._free.append(slot)

    def write(self, layer: int, slot: int, start: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """Store rows [n, Hkv, D] of one layer at positions start ..; the slot's length follows its last layer."""
        n = k.shape[0]
        if start + n > self.max_len:
            raise ValueError(f"slot {slot}: {start + n} tokens exceed max_len {self.max_len}")
        self.k[layer, slot, start:start + n] = k.to(torch.bfloat16)
        self.v[layer, slot, start:start + n] = v.to(torch.bfloat16)
        if layer == self.layers - 1:
            self.lens[slot] = max(self.lens[slot], start + n)


class HeteroAttention:
    """Decode attention over a ``SlotKVStorage`` in mode 0, 1 or 2 (see the module text)."""

    def __init__(self, storage: SlotKVStorage, num_heads: int, mode: int = 1, device="cpu", host_fraction: float = 0.5,
                 threads: int = 8, max_batch: int = 64):
        if mode not in (0, 1, 2):
            raise ValueError("mode is 0 (device), 1 (host) or 2 (split)")
        self.st, self.hq, self.mode, self.threads = storage, num_heads, mode, threads
        self.device = torch.device(device)
        self.host_fraction = host_fraction
        self.scale = storage.d ** -0.5
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.buffers = None
        if mode in (0, 2):
            shape = (2, 2, max_batch, storage.max_len, storage.hkv, storage.d)       # [ping-pong, k|v, rows, ...]
            self.buffers = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
            self._staged = [None, None]                                             # (layer, slots) each buffer holds
            self._events = [None, None]
        self.host_rows = self.device_rows = 0

    # ------------------------------------------------------------------ mode 0: double-buffered device KV
    def prefetch(self, layer: int, slots: Sequence[int], lens: Sequence[int]) -> None:
        """Start copying ``layer``'s KV of the rows into the buffer that is not in use (call it for layer l + 1 before
        computing layer l)."""
        if self.buffers is None or not slots:
            return
        b = layer % 2
        idx = torch.as_tensor(list(slots), dtype=torch.long)
        L = max(lens)
        ctx = torch.cuda.stream(self.copy_stream) if self.copy_stream is not None else _Null()
        with ctx:
            self.buffers[b, 0, :len(slots), :L].copy_(self.st.k[layer, idx, :L], non_blocking=True)
            self.buffers[b, 1, :len(slots), :L].copy_(self.st.v[layer, idx, :L], non_blocking=True)
            if self.copy_stream is not None:
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
                self._events[b] = ev
        self._staged[b] = (layer, tuple(slots))

    def _device_attention(self, layer: int, q: torch.Tensor, slots: Sequence[int], lens: Sequence[int], window: int):
        b = layer % 2
        if self._staged[b] != (layer, tuple(slots)):
            self.prefetch(layer, slots, lens)
        if self._events[b] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._events[b])
        out = torch.empty(len(slots), self.hq, self.st.d, dtype=torch.float32, device=self.device)
        for i, L in enumerate(lens):
            k, v = self.buffers[b, 0, i, :L], self.buffers[b, 1, i, :L]
            out[i] = ref.gqa_attention(q[i:i + 1].to(self.device).float(), k, v, self.scale, q_start=L - 1, window=window)[0]
        return out

    # ------------------------------------------------------------------ mode 1: host attention on the slot memory
    def _host_attention(self, layer: int, q: torch.Tensor, slots: Sequence[int], lens: Sequence[int], window: int):
        from ..core import native
        S = self.st.max_len                                   # the whole slot is one "page" of the paged CPU kernel
        kp = [[self.st.k[layer, s].data_ptr()] for s in slots]
        vp = [[self.st.v[layer, s].data_ptr()] for s in slots]
        return native.cpu_gqa_decode(q.detach().float().cpu(), kp, vp, list(lens), S, self.st.hkv, self.scale,
                                     window=window, threads=self.threads)

    # ------------------------------------------------------------------ entry point
    def decode(self, layer: int, q: torch.Tensor, slots: Sequence[int], lens: Sequence[int], window: int = 0) -> torch.Tensor:
        """q [B, Hq, D] (one query per row, the row's KV up to ``lens[b]`` already written) -> [B, Hq, D] fp32 on the
        query's device."""
        B = q.shape[0]
        if self.mode == 1:
            self.host_rows += B
            return self._host_attention(layer, q, slots, lens, window).to(q.device)
        if self.mode == 0:
            self.device_rows += B
            return self._device_attention(layer, q, slots, lens, window).to(q.device)
        order = sorted(range(B), key=lambda i: -lens[i])
        n_host = int(round(self.host_fraction * B))
        host, dev = sorted(order[:n_host]), sorted(order[n_host:])
        out = torch.empty(B, self.hq, self.st.d, dtype=torch.float32, device=q.device)
        if dev:                                               # enqueue the device part first: the host part overlaps it
            d_out = self._device_attention(layer, q[dev], [slots[i] for i in dev], [lens[i] for i in dev], window)
        if host:
            h_out = self._host_attention(layer, q[host], [slots[i] for i in host], [lens[i] for i in host], window)
            out[host] = h_out.to(q.device)
        if dev:
            out[dev] = d_out.to(q.device)
        self.host_rows += len(host)
        self.device_rows += len(dev)
        return out


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
