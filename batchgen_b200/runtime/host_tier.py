"""Host KV tier on the native engine: a node-shared paged region (memfd) + asynchronous page movers.

``NativeHostTier`` owns (or attaches to) a ``core.native.HostPagedKV`` region whose pages hold one device page of
every layer, layer-major, and moves pages between it and the device pool through ``core.native.KVMover`` on the
mover's own streams.  Every transfer is a *future*: callers get task ids back, order compute after a load with a
device-side wait (no host synchronisation), and return device pages to their allocator only when the offload that
reads them has finished.  The region's prefix coordinator (256-bit hash chain, reference-counted pages) is the second
level of the prefix cache: device pages evicted from ``runtime.prefix_cache.PrefixCache`` are demoted here and
promoted back on a later hit.

Reference parity: core/KV_Storage/host_paged_kv_worker_view.h:386 (async load), :595 (async offload), :870 (futures),
core/KV_Storage/host_prefix_cache_coordinator.h (chain table); the reference keeps host KV primary and appends to it
every decode step (:1064) - here the device pool is primary and pages move when a row is parked or demoted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence as Seq, Tuple

import torch

from ..core import native
from .kv_cache import PagedKVCache


class _HostAlloc:
    """The allocator face the engine expects (``num_free`` / ``alloc`` / ``free``) over the native region."""

    def __init__(self, region: "native.HostPagedKV"):
        self._r = region

    @property
    def num_free(self) -> int:
        return self._r.num_free

    def alloc(self, n: int) -> List[int]:
        if n <= 0:
            return []
        got = self._r.alloc(n)
        if got is None:
            freed = self._r.prefix_evict(n - self._r.num_free)      # cached prefixes yield to live rows
            got = self._r.alloc(n) if freed else None
        if got is None:
            raise MemoryError(f"host KV tier: {n} pages wanted, {self._r.num_free} free")
        return got

    def free(self, pages: Seq[int]) -> None:
        if pages:
            self._r.free(list(pages))


class NativeHostTier:
    """Paged host KV for one worker.  ``fd`` attaches to a region another process created (the server creates one
    per node and hands the descriptor to its workers); otherwise a private region of ``num_pages`` is created."""

    def __init__(self, device_kv: PagedKVCache, num_pages: int = 0, prefix_slots: int = 0, fd: Optional[int] = None,
                 max_fragments: int = 4096):
        if device_kv.device.type != "cuda":
            raise RuntimeError("the native host tier moves pages with CUDA copies: it needs a device pool on a GPU")
        self.dkv = device_kv
        # (device base pointer, bytes per (layer, page) fragment, layers, offset of the group inside a host page)
        self.groups: List[Tuple[int, int, int, int]] = []
        off = 0
        tensors = [device_kv.kv] + ([device_kv.idx_k, device_kv.idx_s] if device_kv.idx_k is not None else [])
        for t in tensors:
            frag = t[0, 0].numel() * t.element_size()
            if frag % 16:
                raise ValueError(f"a page fragment of {frag} bytes is not a multiple of 16")
            self.groups.append((t.data_ptr(), frag, t.shape[0], off))
            off += frag * t.shape[0]
        self.page_bytes = off
        self.pages_per_layer = device_kv.num_pages
        self.region = (native.HostPagedKV(fd=fd) if fd is not None
                       else native.HostPagedKV(num_pages, self.page_bytes, prefix_slots or 2 * num_pages))
        self.region.page_bytes = self.page_bytes
        self.region.pin()
        self.alloc = _HostAlloc(self.region)
        self.max_fragments = max_fragments
        self.mover = native.KVMover(device_kv.device.index or 0, max_fragments=max_fragments, ring=16)
        self.offloaded_pages = self.loaded_pages = self.demoted_pages = self.promoted_pages = 0

    @property
    def num_pages(self) -> int:
        return self.region.num_pages

    # ------------------------------------------------------------------ transfers
    def _fragments(self, gpu_pages: Seq[int], host_pages: Seq[int]):
        """Per fragment size: (device pointers, host pointers) of every (page, layer) fragment."""
        out = []
        hp = [self.region.page_ptr(p) for p in host_pages]
        for base, frag, layers, off in self.groups:
            dev, host = [], []
            for g, h in zip(gpu_pages, hp):
                for l in range(layers):
                    dev.append(base + (l * self.pages_per_layer + g) * frag)
                    host.append(h + off + l * frag)
            out.append((frag, dev, host))
        return out

    def _submit(self, src: List[int], dst: List[int], frag: int, after_stream: Optional[int]) -> List[int]:
        tasks = []
        for i in range(0, len(src), self.max_fragments):
            tasks.append(self.mover.submit(src[i:i + self.max_fragments], dst[i:i + self.max_fragments], frag,
                                           use_kernel=True, after_stream=after_stream))
        return tasks

    def offload(self, gpu_pages: Seq[int], host_pages: Seq[int], after_stream: Optional[int] = None) -> List[int]:
        """Device pages -> host pages, all layers.  ``after_stream``: the copies start after the work already
        enqueued on that stream (the kernels that wrote the KV).  Returns the tasks to wait on."""
        tasks: List[int] = []
        for frag, dev, host in self._fragments(gpu_pages, host_pages):
            tasks += self._submit(dev, host, frag, after_stream)
        self.offloaded_pages += len(gpu_pages)
        return tasks

    def load(self, host_pages: Seq[int], gpu_pages: Seq[int], after_stream: Optional[int] = None) -> List[int]:
        tasks: List[int] = []
        for frag, dev, host in self._fragments(gpu_pages, host_pages):
            tasks += self._submit(host, dev, frag, after_stream)
        self.loaded_pages += len(gpu_pages)
        return tasks

    def done(self, tasks: Seq[int]) -> bool:
        return all(self.mover.done(t) for t in tasks)

    def wait(self, tasks: Seq[int]) -> None:
        for t in tasks:
            self.mover.wait(t)

    def stream_wait(self, tasks: Seq[int], stream: int) -> None:
        """Order ``stream`` after the transfers (device-side; the host does not block)."""
        for t in tasks:
            self.mover.stream_wait(t, stream)

    # ------------------------------------------------------------------ second-level prefix cache
    def demote(self, key: bytes, gpu_page: int, after_stream: Optional[int] = None) -> Optional[List[int]]:
        """Keep a prefix page that leaves the device cache: copy it into a host page published under ``key``.
        Returns the copy's tasks (the device page may be reused once they are done) or None when the host tier has
        no room."""
        if self.region.num_free == 0 and self.region.prefix_evict(1) == 0:
            return None
        got = self.region.alloc(1)
        if got is None:
            return None
        tasks = self.offload([gpu_page], got, after_stream)
        self.region.L.bgc_prefix_commit(self.region.h, key, (native.ctypes.c_int * 1)(got[0]), 1)
        self.region.free(got)                   # the coordinator keeps its own reference
        self.demoted_pages += 1
        return tasks

    def lookup(self, keys: Seq[bytes]) -> List[int]:
        """Host pages for the longest run of ``keys`` (chain keys of consecutive pages) present in the coordinator;
        a reference is taken for the caller on each (release with ``alloc.free``)."""
        if not keys:
            return []
        n = len(keys)
        out = (native.ctypes.c_int * n)()
        m = self.region.L.bgc_prefix_lookup_attach(self.region.h, b"".join(keys), n, out)
        return list(out)[:m]

    def stats(self) -> Dict[str, int]:
        d = dict(offloaded_pages=self.offloaded_pages, loaded_pages=self.loaded_pages,
                 demoted_pages=self.demoted_pages, promoted_pages=self.promoted_pages,
                 bytes_moved=self.mover.bytes_moved, host_pages_free=self.region.num_free)
        d.update({f"prefix_{k}": v for k, v in self.region.prefix_stats().items()})
        return d

    def close(self) -> None:
        self.mover.close()
        self.region.close()
