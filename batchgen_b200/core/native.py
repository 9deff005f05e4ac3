"""ctypes front of the native engine (``batchgen_b200/_C/libbg_core.so``): weight ring, node-shared host
paged KV with its prefix coordinator, KV page movers and the CPU decode-attention kernel.

The library is C++ (``core/csrc``), built in-tree by ``batchgen_b200.build``.  Everything except the CUDA copy
backend and the page movers works without a GPU, which is how these classes are tested.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

_LIB: Optional[ctypes.CDLL] = None
_PATH = Path(__file__).resolve().parent.parent / "_C" / "libbg_core.so"


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not _PATH.exists():
            from .. import build
            build.build_core()
        L = ctypes.CDLL(str(_PATH))
        L.bgc_ring_create.restype = ctypes.c_void_p
        L.bgc_ring_get.restype = ctypes.c_void_p
        L.bgc_ring_begin_pass.restype = ctypes.c_ulonglong
        L.bgc_hostkv_create.restype = ctypes.c_void_p
        L.bgc_hostkv_attach.restype = ctypes.c_void_p
        L.bgc_hostkv_page_ptr.restype = ctypes.c_void_p
        L.bgc_hostkv_base.restype = ctypes.c_void_p
        L.bgc_hostkv_num_free.restype = ctypes.c_ulonglong
        L.bgc_hostkv_num_pages.restype = ctypes.c_ulonglong
        L.bgc_hostkv_bytes.restype = ctypes.c_ulonglong
        L.bgc_mover_create.restype = ctypes.c_void_p
        for f in ("bgc_wd_staging_bytes", "bgc_wd_epoch", "bgc_wd_begin_swap"):
            getattr(L, f).restype = ctypes.c_ulonglong
        for f in ("bgc_swa_create", "bgc_cratio_create", "bgc_wd_create", "bgc_wdc_create"):
            getattr(L, f).restype = ctypes.c_void_p
        for f in ("bgc_swa_advance", "bgc_swa_append_position", "bgc_swa_write_rows", "bgc_swa_read_window",
                  "bgc_cratio_offload", "bgc_cratio_append", "bgc_cratio_read"):
            getattr(L, f).restype = ctypes.c_long
        for f in ("bgc_swa_active_pages", "bgc_swa_window_start", "bgc_cratio_stored", "bgc_cratio_pages"):
            getattr(L, f).restype = ctypes.c_ulonglong
        L.bgc_mover_submit.restype = ctypes.c_long
        L.bgc_mover_bytes.restype = ctypes.c_ulonglong
        L.bgc_mover_misaligned.restype = ctypes.c_ulonglong
        _LIB = L
    return _LIB


SLOT_STATES = {"FREE": 0, "FILLING": 1, "PRESENT": 2, "LEASED": 3, "PENDING_RELEASE": 4}


class WeightRing:
    """Ring of device weight slots fed from host memory by a native producer thread.

    ``modules`` maps a module key (e.g. ``routed_expert_5_17``) to its host tensors; ``get(key)`` blocks until
    the module is resident and returns tensors viewing the slot; ``release(key)`` hands the slot back."""

    def __init__(self, num_slots: int, slot_bytes: int, device: str = "cpu"):
        self.L = lib()
        self.device = torch.device(device)
        backend = 1 if self.device.type == "cuda" else 0
        self.h = ctypes.c_void_p(self.L.bgc_ring_create(num_slots, ctypes.c_ulonglong(slot_bytes), backend,
                                                        self.device.index or 0))
        if not self.h:
            raise RuntimeError("could not create the weight ring (CUDA backend unavailable?)")
        self.slot_bytes = slot_bytes
        self.ids: Dict[str, int] = {}
        self.layout: Dict[int, List[Tuple[str, torch.dtype, Tuple[int, ...], int]]] = {}
        self._host_refs: Dict[int, List[torch.Tensor]] = {}
        self._leases: Dict[str, int] = {}

    def register(self, key: str, tensors: Dict[str, torch.Tensor]) -> None:
        mid = self.ids.setdefault(key, len(self.ids))
        names = list(tensors)
        ts = [tensors[n].contiguous() for n in names]
        for t in ts:
            assert t.device.type == "cpu", "streamed weights live in host memory"
        n = len(ts)
        ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
        sizes = (ctypes.c_ulonglong * n)(*[t.numel() * t.element_size() for t in ts])
        offs = (ctypes.c_ulonglong * n)()
        if self.L.bgc_ring_register_module(self.h, mid, ptrs, sizes, n, offs) != 0:
            raise ValueError(f"module {key} does not fit a slot of {self.slot_bytes} bytes")
        self.layout[mid] = [(names[i], ts[i].dtype, tuple(ts[i].shape), int(offs[i])) for i in range(n)]
        self._host_refs[mid] = ts

    def install_queue(self, keys: Sequence[str]) -> None:
        arr = (ctypes.c_int * len(keys))(*[self.ids[k] for k in keys])
        self.L.bgc_ring_install_queue(self.h, arr, len(keys))

    def begin_pass(self, carry: bool = False) -> int:
        return int(self.L.bgc_ring_begin_pass(self.h, int(carry)))

    def end_pass(self) -> bool:
        return self.L.bgc_ring_end_pass(self.h) == 0

    def skip(self, keys: Sequence[str]) -> None:
        arr = (ctypes.c_int * len(keys))(*[self.ids[k] for k in keys])
        self.L.bgc_ring_skip(self.h, arr, len(keys))

    def abort(self) -> None:
        self.L.bgc_ring_abort(self.h)
        self._leases.clear()

    def start(self) -> None:
        self.L.bgc_ring_start(self.h)

    def stop(self) -> None:
        self.L.bgc_ring_stop(self.h)

    def get(self, key: str, timeout_ms: int = 300_000) -> Optional[Dict[str, torch.Tensor]]:
        mid = self.ids[key]
        slot = ctypes.c_int(-1)
        p = self.L.bgc_ring_get(self.h, mid, timeout_ms, ctypes.byref(slot))
        if not p:
            return None
        self._leases[key] = slot.value
        out = {}
        for name, dt, shape, off in self.layout[mid]:
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty(0, dtype=dt).element_size()
            if self.device.type == "cuda":
                out[name] = _cuda_view(p + off, nbytes, dt, shape, self.device)
            else:
                buf = (ctypes.c_char * nbytes).from_address(p + off)
                out[name] = torch.frombuffer(buf, dtype=torch.uint8).view(dt).view(*shape)
        return out

    def release(self, key: str, stream: Optional[int] = None) -> None:
        slot = self._leases.pop(key)
        self.L.bgc_ring_release(self.h, slot, ctypes.c_void_p(stream or 0))

    def count(self, state: str) -> int:
        return self.L.bgc_ring_count_state(self.h, SLOT_STATES[state])

    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_ulonglong * 7)()
        self.L.bgc_ring_stats(self.h, out)
        k = ["modules_copied", "modules_skipped", "bytes_copied", "get_calls", "get_wait_us", "stalls", "copy_us"]
        return dict(zip(k, [int(v) for v in out]))

    def close(self) -> None:
        if self.h:
            self.L.bgc_ring_destroy(self.h)
            self.h = None


def _cuda_view(ptr: int, nbytes: int, dtype, shape, device) -> torch.Tensor:
    """A torch tensor over raw device memory owned by the native ring (CUDA array interface)."""
    class _Holder:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
    return torch.as_tensor(_Holder(), device=device).view(dtype).view(*shape)


def prefix_keys(token_ids: Sequence[int], page_size: int, salt: bytes = b"") -> bytes:
    """The 256-bit hash chain over full pages of ``token_ids`` (same chain as runtime.prefix_cache)."""
    from ..runtime.prefix_cache import build_prefix_hash_chain
    return b"".join(build_prefix_hash_chain(token_ids, page_size, salt))


class HostPagedKV:
    """Node-shared paged host KV region (memfd) with the prefix coordinator inside."""

    def __init__(self, num_pages: int = 0, page_bytes: int = 0, prefix_slots: int = 0, fd: Optional[int] = None):
        self.L = lib()
        if fd is None:
            out = ctypes.c_int(-1)
            self.h = ctypes.c_void_p(self.L.bgc_hostkv_create(ctypes.c_ulonglong(num_pages), ctypes.c_ulonglong(page_bytes),
                                                              ctypes.c_ulonglong(prefix_slots), ctypes.byref(out)))
            self.fd = out.value
        else:
            self.h = ctypes.c_void_p(self.L.bgc_hostkv_attach(fd))
            self.fd = fd
        if not self.h:
            raise RuntimeError("could not create / attach the host KV region")
        self.page_bytes = page_bytes
        self._pinned = False

    @property
    def num_pages(self) -> int:
        return int(self.L.bgc_hostkv_num_pages(self.h))

    @property
    def num_free(self) -> int:
        return int(self.L.bgc_hostkv_num_free(self.h))

    def alloc(self, n: int) -> Optional[List[int]]:
        out = (ctypes.c_int * n)()
        return list(out) if self.L.bgc_hostkv_alloc(self.h, n, out) == 0 else None

    def share(self, pages: Sequence[int]) -> None:
        self.L.bgc_hostkv_share(self.h, (ctypes.c_int * len(pages))(*pages), len(pages))

    def free(self, pages: Sequence[int]) -> None:
        self.L.bgc_hostkv_free(self.h, (ctypes.c_int * len(pages))(*pages), len(pages))

    def refcount(self, page: int) -> int:
        return self.L.bgc_hostkv_refcount(self.h, page)

    def page_ptr(self, page: int) -> int:
        return int(self.L.bgc_hostkv_page_ptr(self.h, page))

    def page_tensor(self, page: int, dtype=torch.uint8) -> torch.Tensor:
        buf = (ctypes.c_char * self.page_bytes).from_address(self.page_ptr(page))
        return torch.frombuffer(buf, dtype=torch.uint8).view(dtype)

    def audit(self) -> int:
        return self.L.bgc_hostkv_audit(self.h)

    def pin(self) -> bool:
        """Register the mapping with CUDA so that pages can be sources / targets of async copies."""
        if not self._pinned and torch.cuda.is_available():
            rc = self.L.bgc_pin_host(ctypes.c_void_p(self.L.bgc_hostkv_base(self.h)),
                                     ctypes.c_size_t(self.L.bgc_hostkv_bytes(self.h)))
            self._pinned = rc == 0
        return self._pinned

    # ---- prefix coordinator
    def prefix_commit(self, token_ids: Sequence[int], pages: Sequence[int], page_size: int) -> int:
        keys = prefix_keys(token_ids, page_size)
        n = min(len(keys) // 32, len(pages))
        return self.L.bgc_prefix_commit(self.h, keys, (ctypes.c_int * n)(*pages[:n]), n)

    def prefix_lookup_attach(self, token_ids: Sequence[int], page_size: int) -> List[int]:
        keys = prefix_keys(token_ids[: max(len(token_ids) - 1, 0)], page_size)
        n = len(keys) // 32
        out = (ctypes.c_int * max(n, 1))()
        m = self.L.bgc_prefix_lookup_attach(self.h, keys, n, out)
        return list(out)[:m]

    def prefix_evict(self, want: int) -> int:
        return self.L.bgc_prefix_evict(self.h, want)

    def prefix_clear(self) -> int:
        return self.L.bgc_prefix_clear(self.h)

    def prefix_stats(self) -> Dict[str, int]:
        out = (ctypes.c_ulonglong * 4)()
        self.L.bgc_prefix_stats(self.h, out)
        return dict(zip(["entries", "hits", "misses", "evicted"], [int(v) for v in out]))

    def close(self) -> None:
        if self.h:
            if self._pinned:                      # registrations do not go away with the mapping
                self.L.bgc_unpin_host(ctypes.c_void_p(self.L.bgc_hostkv_base(self.h)))
                self._pinned = False
            self.L.bgc_hostkv_destroy(self.h)
            self.h = None


class _RowView:
    """Shared plumbing of the per-sequence row views: rows are fixed-size token records of one layer."""

    def __init__(self, kv: HostPagedKV, row_shape: Sequence[int], dtype: torch.dtype):
        self.kv, self.L = kv, kv.L
        self.row_shape, self.dtype = tuple(row_shape), dtype
        n = 1
        for d in self.row_shape:
            n *= d
        self.row_bytes = n * torch.empty(0, dtype=dtype).element_size()

    def _rows_ptr(self, rows: torch.Tensor):
        assert rows.dtype == self.dtype and rows.is_contiguous() and not rows.is_cuda
        assert tuple(rows.shape[1:]) == self.row_shape, (rows.shape, self.row_shape)
        return ctypes.c_void_p(rows.data_ptr())

    def _out(self, n: int) -> torch.Tensor:
        return torch.empty((n,) + self.row_shape, dtype=self.dtype)

    @staticmethod
    def _check(rc: int, what: str) -> int:
        if rc == -2:
            raise MemoryError(f"{what}: the host KV region has no free page")
        if rc == -3:
            raise RuntimeError(f"{what}: a stored position has no page")
        return rc


class SlidingWindowHostView(_RowView):
    """Host KV of sliding-window layers: a sequence holds only the pages that overlap its last ``window`` tokens
    (at most window / page + 1); older pages return to the region as the sequence grows.

    Reference parity: core/KV_Storage/swa_host_paged_kv_worker_view.h."""

    def __init__(self, kv: HostPagedKV, page_tokens: int, layers: int, row_shape: Sequence[int], dtype: torch.dtype,
                 window_tokens: int):
        super().__init__(kv, row_shape, dtype)
        self.h = ctypes.c_void_p(self.L.bgc_swa_create(kv.h, page_tokens, self.row_bytes, layers,
                                                       ctypes.c_ulonglong(window_tokens)))
        if not self.h:
            raise ValueError("window must be a positive multiple of the page size and a page must hold "
                             "layers x page_tokens rows")
        self.window = window_tokens

    def write(self, seq: int, layer: int, raw_start: int, rows: torch.Tensor) -> int:
        """Store rows of raw positions raw_start ..; rows that already fell out of the window are skipped.  Raises
        ``IndexError`` for a range older than the kept window."""
        rc = self.L.bgc_swa_write_rows(self.h, ctypes.c_longlong(seq), layer, ctypes.c_ulonglong(raw_start),
                                       self._rows_ptr(rows), ctypes.c_ulonglong(rows.shape[0]))
        if rc == -1:
            raise IndexError("rows older than the sliding window cannot be written")
        return self._check(rc, "SlidingWindowHostView.write")

    def append_position(self, seq: int, raw_pos: int) -> int:
        rc = self.L.bgc_swa_append_position(self.h, ctypes.c_longlong(seq), ctypes.c_ulonglong(raw_pos))
        if rc == -1:
            raise IndexError("position older than the sliding window")
        return self._check(rc, "SlidingWindowHostView.append_position")

    def read(self, seq: int, layer: int) -> Tuple[torch.Tensor, int]:
        """-> (rows of the window, oldest first; raw position of the first row)."""
        out = self._out(self.window)
        first = ctypes.c_ulonglong(0)
        n = self._check(self.L.bgc_swa_read_window(self.h, ctypes.c_longlong(seq), layer, ctypes.c_void_p(out.data_ptr()),
                                                   ctypes.c_ulonglong(self.window), ctypes.byref(first)), "read")
        return out[:n], int(first.value)

    def active_pages(self, seq: int) -> int:
        return int(self.L.bgc_swa_active_pages(self.h, ctypes.c_longlong(seq)))

    def window_start(self, seq: int) -> int:
        return int(self.L.bgc_swa_window_start(self.h, ctypes.c_longlong(seq)))

    def release(self, seq: int) -> None:
        self.L.bgc_swa_release(self.h, ctypes.c_longlong(seq))

    def close(self) -> None:
        if self.h:
            self.L.bgc_swa_destroy(self.h)
            self.h = None


class CompressedRatioHostView(_RowView):
    """Host KV of compressed layers: one stored row per ``ratio`` raw tokens; a decode step stores a row only when
    its position closes a group of ``ratio``.

    Reference parity: core/KV_Storage/compressed_ratio_host_paged_kv_worker_view.h."""

    def __init__(self, kv: HostPagedKV, page_tokens: int, layers: int, row_shape: Sequence[int], dtype: torch.dtype,
                 ratio: int):
        super().__init__(kv, row_shape, dtype)
        self.h = ctypes.c_void_p(self.L.bgc_cratio_create(kv.h, page_tokens, self.row_bytes, layers, ctypes.c_ulonglong(ratio)))
        if not self.h:
            raise ValueError("ratio must be positive and a page must hold layers x page_tokens rows")
        self.ratio = ratio

    def offload(self, seq: int, layer: int, raw_len: int, rows: torch.Tensor) -> int:
        """Store the ``raw_len // ratio`` pooled rows of a prefilled sequence."""
        assert rows.shape[0] >= raw_len // self.ratio
        return self._check(self.L.bgc_cratio_offload(self.h, ctypes.c_longlong(seq), layer, ctypes.c_ulonglong(raw_len),
                                                     self._rows_ptr(rows)), "CompressedRatioHostView.offload")

    def append(self, seq: int, layer: int, raw_pos: int, row: torch.Tensor) -> int:
        """Decode step at ``raw_pos``: -> the storage position written, or -1 when the position closes no group."""
        return self._check(self.L.bgc_cratio_append(self.h, ctypes.c_longlong(seq), layer, ctypes.c_ulonglong(raw_pos),
                                                    self._rows_ptr(row.reshape((1,) + self.row_shape))), "append")

    def read(self, seq: int, layer: int) -> torch.Tensor:
        n = self.stored(seq)
        out = self._out(n)
        got = self._check(self.L.bgc_cratio_read(self.h, ctypes.c_longlong(seq), layer, ctypes.c_void_p(out.data_ptr()),
                                                 ctypes.c_ulonglong(n)), "read")
        return out[:got]

    def stored(self, seq: int) -> int:
        return int(self.L.bgc_cratio_stored(self.h, ctypes.c_longlong(seq)))

    def pages(self, seq: int) -> int:
        return int(self.L.bgc_cratio_pages(self.h, ctypes.c_longlong(seq)))

    def release(self, seq: int) -> None:
        self.L.bgc_cratio_release(self.h, ctypes.c_longlong(seq))

    def close(self) -> None:
        if self.h:
            self.L.bgc_cratio_destroy(self.h)
            self.h = None


class KVMover:
    """Asynchronous page gather/scatter between pinned host memory and device memory (GPU only)."""

    def __init__(self, device: int = 0, max_fragments: int = 4096, ring: int = 8):
        self.L = lib()
        self.h = ctypes.c_void_p(self.L.bgc_mover_create(device, max_fragments, ring))
        if not self.h:
            raise RuntimeError("KVMover needs a CUDA device")

    def submit(self, src_ptrs: Sequence[int], dst_ptrs: Sequence[int], nbytes: int, use_kernel: bool = True,
               after_stream: Optional[int] = None) -> int:
        n = len(src_ptrs)
        s = (ctypes.c_void_p * n)(*src_ptrs)
        d = (ctypes.c_void_p * n)(*dst_ptrs)
        t = self.L.bgc_mover_submit(self.h, s, d, n, ctypes.c_size_t(nbytes), int(use_kernel),
                                    ctypes.c_void_p(after_stream or 0))
        if t < 0:
            raise RuntimeError(f"mover refused the request ({t})")
        return int(t)

    def done(self, task: int) -> bool:
        return self.L.bgc_mover_done(self.h, ctypes.c_long(task)) == 1

    def wait(self, task: int) -> None:
        self.L.bgc_mover_wait(self.h, ctypes.c_long(task))

    def stream_wait(self, task: int, stream: int) -> None:
        self.L.bgc_mover_stream_wait(self.h, ctypes.c_long(task), ctypes.c_void_p(stream))

    @property
    def bytes_moved(self) -> int:
        return int(self.L.bgc_mover_bytes(self.h))

    @property
    def misaligned_fallbacks(self) -> int:
        """Kernel-path requests that went to the copy engine because a fragment was not 16-byte aligned."""
        return int(self.L.bgc_mover_misaligned(self.h))

    def close(self) -> None:
        if self.h:
            self.L.bgc_mover_destroy(self.h)
            self.h = None


def cpu_gqa_decode(q: torch.Tensor, k_pages: Sequence[Sequence[int]], v_pages: Sequence[Sequence[int]],
                   lens: Sequence[int], page_size: int, num_kv_heads: int, scale: float, window: int = 0,
                   threads: int = 8) -> torch.Tensor:
    """q [B, Hq, D] fp32; k/v page *addresses* per sequence (bf16 pages [page, Hkv, D]) -> [B, Hq, D] fp32."""
    B, Hq, D = q.shape
    q = q.contiguous().float()
    out = torch.empty_like(q)
    mp = max(len(p) for p in k_pages)
    kp = (ctypes.c_void_p * (B * mp))()
    vp = (ctypes.c_void_p * (B * mp))()
    for b in range(B):
        for i, a in enumerate(k_pages[b]):
            kp[b * mp + i] = a
        for i, a in enumerate(v_pages[b]):
            vp[b * mp + i] = a
    ln = (ctypes.c_int * B)(*lens)
    rc = lib().bgc_cpu_gqa_decode(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(out.data_ptr()), kp, vp, ln, B, mp,
                                  page_size, Hq, num_kv_heads, D, ctypes.c_float(scale), window, threads)
    if rc != 0:
        raise ValueError("bad GQA geometry")
    return out


class ParameterStore:
    """Node-shared weight region: the server creates it and loads converted checkpoint shards into it with
    parallel readers; workers attach by descriptor and read tensors as views (optionally pinned for DMA).

    Reference parity: core/Parameter_Server/Parameter_Server.cpp (allocate + read), core/Weights_Storage/
    Weights_Storage.h:70-178 (worker-side attach, cudaHostRegister, per-module tensor map)."""

    def __init__(self, nbytes: int = 0, fd: Optional[int] = None, huge_pages: bool = True, read_only: bool = False):
        L = lib()
        L.bgc_pstore_create.restype = ctypes.c_void_p
        L.bgc_pstore_attach.restype = ctypes.c_void_p
        L.bgc_pstore_base.restype = ctypes.c_void_p
        L.bgc_pstore_bytes.restype = ctypes.c_ulonglong
        if fd is None:
            out = ctypes.c_int(-1)
            self._h = L.bgc_pstore_create(ctypes.c_ulonglong(nbytes), ctypes.c_int(int(huge_pages)), ctypes.byref(out))
            self.fd = out.value
        else:
            self._h = L.bgc_pstore_attach(ctypes.c_int(fd), ctypes.c_int(int(read_only)))
            self.fd = fd
        if not self._h:
            raise MemoryError("parameter store: could not create or attach the shared region")
        self.nbytes = int(L.bgc_pstore_bytes(ctypes.c_void_p(self._h)))
        self.base = int(L.bgc_pstore_base(ctypes.c_void_p(self._h)))
        self.index: Dict[str, Tuple[int, torch.dtype, Tuple[int, ...]]] = {}
        self._pinned = False

    def load_converted(self, ckpt_dir: str, threads: int = 8) -> int:
        """Read every ``*.bin`` shard of a converted checkpoint (see ``ckpt.converter``) back to back into the
        region and index its tensors.  Returns the bytes loaded."""
        import glob
        import json
        import os
        metas = sorted(glob.glob(os.path.join(ckpt_dir, "*.json")))
        paths, offs, sizes = [], [], []
        cur = 0
        for m in metas:
            with open(m) as f:
                meta = json.load(f)
            if "total_byte_size" not in meta:           # not a shard description (e.g. a staging manifest)
                continue
            n = int(meta["total_byte_size"])
            paths.append(os.path.join(ckpt_dir, meta["file_name"]).encode())
            offs.append(cur)
            sizes.append(n)
            for name, t in meta["state_dict"].items():
                self.index[name] = (cur + int(t["offset"]), getattr(torch, t["dtype"].replace("torch.", "")), tuple(t["shape"]))
            cur += (n + 255) // 256 * 256
        if cur > self.nbytes:
            raise MemoryError(f"checkpoint needs {cur} bytes, the store holds {self.nbytes}")
        arr = (ctypes.c_char_p * len(paths))(*paths)
        o = (ctypes.c_ulonglong * len(paths))(*offs)
        z = (ctypes.c_ulonglong * len(paths))(*sizes)
        rc = lib().bgc_pstore_load_files(ctypes.c_void_p(self._h), arr, o, z, ctypes.c_int(len(paths)), ctypes.c_int(threads))
        if rc != 0:
            raise OSError(f"parameter store: reading {paths[-rc - 1].decode()} failed")
        return sum(sizes)

    @staticmethod
    def bytes_needed(ckpt_dir: str) -> int:
        import glob
        import json
        import os
        total = 0
        for m in sorted(glob.glob(os.path.join(ckpt_dir, "*.json"))):
            with open(m) as f:
                total += (int(json.load(f).get("total_byte_size", 0)) + 255) // 256 * 256
        return total

    def export_index(self) -> Dict[str, Tuple[int, str, Tuple[int, ...]]]:
        return {k: (o, str(d), s) for k, (o, d, s) in self.index.items()}

    def import_index(self, idx) -> None:
        self.index = {k: (o, getattr(torch, d.replace("torch.", "")), tuple(s)) for k, (o, d, s) in idx.items()}

    def tensor(self, name: str) -> torch.Tensor:
        off, dtype, shape = self.index[name]
        n = 1
        for v in shape:
            n *= v
        buf = (ctypes.c_char * (n * torch.empty(0, dtype=dtype).element_size())).from_address(self.base + off)
        return torch.frombuffer(buf, dtype=dtype, count=n).view(*shape)

    def loader(self):
        """``WeightSource`` loader: name, shape -> tensor view or None."""
        def load(name, shape):
            return self.tensor(name) if name in self.index else None
        return load

    def pin(self) -> bool:
        if not torch.cuda.is_available() or self._pinned:
            return self._pinned
        self._pinned = lib().bgc_pin_host(ctypes.c_void_p(self.base), ctypes.c_ulonglong(self.nbytes)) == 0
        return self._pinned

    def close(self) -> None:
        if self._h:
            if self._pinned:
                lib().bgc_unpin_host(ctypes.c_void_p(self.base))
            lib().bgc_pstore_destroy(ctypes.c_void_p(self._h))
            self._h = None


class ReplicaControlBlock:
    """Shared-memory barrier words of a weight replica group (owner publishes a frame -> readers pull ->
    readers acknowledge -> owner reuses the slot), with abort flags and bounded waits."""
    OK, TIMEOUT, ABORTED = 0, 1, 2

    def __init__(self, store: ParameterStore, offset: int, members: int, init: bool):
        L = lib()
        L.bgc_rcb_bytes.restype = ctypes.c_ulonglong
        L.bgc_rcb_slot_frame.restype = ctypes.c_ulonglong
        self.nbytes = int(L.bgc_rcb_bytes())
        if offset % 64 or offset + self.nbytes > store.nbytes:
            raise ValueError("control block must be 64-byte aligned inside the shared region")
        self._mem = ctypes.c_void_p(store.base + offset)
        self._store = store
        if init and L.bgc_rcb_init(self._mem, ctypes.c_int(members)) != 0:
            raise ValueError("replica control block: bad member count")

    @staticmethod
    def size() -> int:
        L = lib()
        L.bgc_rcb_bytes.restype = ctypes.c_ulonglong
        return int(L.bgc_rcb_bytes())

    def publish(self, member: int, mtype: int, slot: int, frame: int) -> None:
        if lib().bgc_rcb_publish(self._mem, member, mtype, slot, ctypes.c_ulonglong(frame)) != 0:
            raise ValueError("publish: bad arguments or uninitialised block")

    def wait_published(self, owner: int, mtype: int, frame: int, timeout_ms: int = 300_000) -> int:
        return lib().bgc_rcb_wait_published(self._mem, owner, mtype, ctypes.c_ulonglong(frame), timeout_ms)

    def ack_pulled(self, member: int, mtype: int, frame: int) -> None:
        lib().bgc_rcb_ack_pulled(self._mem, member, mtype, ctypes.c_ulonglong(frame))

    def wait_all_pulled(self, owner: int, mtype: int, frame: int, timeout_ms: int = 300_000) -> int:
        return lib().bgc_rcb_wait_all_pulled(self._mem, owner, mtype, ctypes.c_ulonglong(frame), timeout_ms)

    def slot_frame(self, member: int, slot: int) -> int:
        return int(lib().bgc_rcb_slot_frame(self._mem, member, slot))

    def abort(self, member: int) -> None:
        lib().bgc_rcb_abort(self._mem, member)


class WeightDaemon:
    """Node daemon of a distributed host weight store: serves this node's share of the modules to the other nodes,
    keeps remote modules that the schedule needs next in a staging region, and leases them to the node's workers over
    a unix socket (``WeightDaemonClient``).

    Reference parity: core/Weights_Storage/distributed_weight_daemon.{h,cpp} (UCX RMA there; a TCP stream here)."""

    def __init__(self, node: int, socket_path: str, listen_port: int = 0, peers: Optional[Dict[int, str]] = None,
                 staging_slots: int = 4, slot_bytes: int = 0, prefetch_depth: int = 2, acquire_wait_ms: int = 50):
        self.L = lib()
        peer_s = ",".join(f"{n}={a}" for n, a in (peers or {}).items())
        self.h = ctypes.c_void_p(self.L.bgc_wd_create(node, socket_path.encode(), listen_port, peer_s.encode(), staging_slots,
                                                      ctypes.c_ulonglong(slot_bytes), prefetch_depth, acquire_wait_ms))
        self.node, self.socket_path, self.slot_bytes = node, socket_path, slot_bytes
        self._store = None
        self._staging = None

    def set_local_store(self, store: torch.Tensor) -> None:
        """``store``: a contiguous uint8 host tensor holding this node's modules back to back (kept alive here)."""
        assert store.dtype == torch.uint8 and store.is_contiguous() and not store.is_cuda
        self._store = store
        self.L.bgc_wd_set_store(self.h, ctypes.c_void_p(store.data_ptr()), ctypes.c_ulonglong(store.numel()))

    def add_module(self, key: str, owner: int, offset: int, nbytes: int) -> None:
        if self.L.bgc_wd_add_module(self.h, key.encode(), owner, ctypes.c_ulonglong(offset), ctypes.c_ulonglong(nbytes)) != 0:
            raise ValueError(f"module {key!r}: outside the local store, larger than a staging slot, or a bad key")

    def set_schedule(self, keys: Sequence[str]) -> None:
        self.L.bgc_wd_set_schedule(self.h, "\n".join(keys).encode())

    def start(self) -> None:
        if self.L.bgc_wd_start(self.h) != 0:
            raise RuntimeError("the weight daemon could not open its sockets or staging region")

    def staging(self) -> torch.Tensor:
        """The staging region as a uint8 tensor (a second mapping of the daemon's memfd, as a worker would make)."""
        if self._staging is None:
            import mmap
            n = int(self.L.bgc_wd_staging_bytes(self.h))
            self._mm = mmap.mmap(self.L.bgc_wd_staging_fd(self.h), n, mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
            self._staging = torch.frombuffer(self._mm, dtype=torch.uint8)
        return self._staging

    @property
    def epoch(self) -> int:
        return int(self.L.bgc_wd_epoch(self.h))

    def begin_swap(self) -> int:
        return int(self.L.bgc_wd_begin_swap(self.h))

    def _json(self, fn) -> Dict:
        import json
        buf = ctypes.create_string_buffer(4096)
        fn(self.h, buf, 4096)
        return json.loads(buf.value.decode())

    def finish_swap(self) -> Dict:
        return self._json(self.L.bgc_wd_finish_swap)

    def status(self) -> Dict:
        return self._json(self.L.bgc_wd_status)

    def stop(self) -> None:
        if self.h:
            self._staging = None
            if getattr(self, "_mm", None) is not None:
                try:
                    self._mm.close()
                except BufferError:
                    pass
                self._mm = None
            self.L.bgc_wd_stop(self.h)
            self.L.bgc_wd_destroy(self.h)
            self.h = None


class WeightDaemonClient:
    """Worker side: ``acquire`` returns ("local", offset, bytes) for a module of this node's store or
    ("staging", offset, bytes) with a lease on a staging slot; ``release`` gives the lease back."""

    def __init__(self, socket_path: str, worker: int, epoch: int):
        self.L = lib()
        self.h = ctypes.c_void_p(self.L.bgc_wdc_create())
        if self.L.bgc_wdc_connect(self.h, socket_path.encode()) != 0:
            raise ConnectionError(f"no weight daemon at {socket_path}")
        rc = self.L.bgc_wdc_hello(self.h, worker, ctypes.c_ulonglong(epoch))
        if rc != 0:
            raise PermissionError(f"weight daemon refused the hello: {self._error()}")

    def _error(self) -> str:
        buf = ctypes.create_string_buffer(256)
        self.L.bgc_wdc_error(self.h, buf, 256)
        return buf.value.decode()

    def acquire(self, key: str, timeout_ms: int = 300_000) -> Tuple[str, int, int]:
        slot, off, nb = ctypes.c_int(-1), ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
        rc = self.L.bgc_wdc_acquire(self.h, key.encode(), timeout_ms, ctypes.byref(slot), ctypes.byref(off), ctypes.byref(nb))
        if rc == 1:
            raise TimeoutError(f"module {key!r} was not ready within {timeout_ms} ms")
        if rc != 0:
            raise RuntimeError(f"acquire({key!r}) failed: {self._error()}")
        return ("local" if slot.value < 0 else "staging"), int(off.value), int(nb.value)

    def release(self, key: str) -> None:
        rc = self.L.bgc_wdc_release(self.h, key.encode())
        if rc not in (0, -6):
            raise RuntimeError(f"release({key!r}) failed: {self._error()}")

    def close(self) -> None:
        if self.h:
            self.L.bgc_wdc_close(self.h)
            self.L.bgc_wdc_destroy(self.h)
            self.h = None


class DistributedModuleSource:
    """Worker-side view of a weight store that is spread over nodes: a module is read straight from this node's local
    store when it lives here, otherwise through a lease on the node daemon's staging region (``WeightDaemonClient``).
    ``module(key)`` returns a uint8 tensor view plus a release callable; the view is valid until released.

    Reference parity: core/Weights_Storage/Weights_Storage.h:70-178 (distributed mode: node daemon socket + leases)."""

    def __init__(self, local_store: torch.Tensor, staging: torch.Tensor, client: "WeightDaemonClient"):
        assert local_store.dtype == torch.uint8 and staging.dtype == torch.uint8
        self.local, self.staging, self.client = local_store, staging, client
        self.local_reads = self.remote_reads = 0

    def module(self, key: str, timeout_ms: int = 300_000):
        where, off, nb = self.client.acquire(key, timeout_ms)
        if where == "local":
            self.local_reads += 1
            return self.local[off: off + nb], (lambda: None)
        self.remote_reads += 1
        return self.staging[off: off + nb], (lambda: self.client.release(key))

    def tensor(self, key: str, dtype: torch.dtype, shape: Sequence[int], timeout_ms: int = 300_000) -> torch.Tensor:
        """A private copy of the module as a typed tensor (the lease is given back before returning)."""
        view, release = self.module(key, timeout_ms)
        try:
            return view.clone().view(dtype).view(*shape)
        finally:
            release()
