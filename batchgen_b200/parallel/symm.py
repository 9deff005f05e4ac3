"""Symmetric heap over NVLink: one allocation per rank, mapped into every peer.

``torch.distributed._symmetric_memory`` does the plumbing (CUDA VMM allocation, handle exchange over the
process group's store, peer mapping); this class carves the allocation into named regions with a bump
allocator that is identical on every rank, so that *region offset + peer base* addresses the same
object on any GPU.  Kernels receive ``peer_ptrs(region)`` — up to 8 raw device pointers — and issue
plain loads/stores to them; nothing here goes through NCCL.

Reference parity: the reference exports VMM ring segments as POSIX fds and maps them into peers for
its weight-replica pulls (core/GPU_Weight_Buffer/vmm_ring_segment.h:1-80) and relies on NVSHMEM heaps
inside DeepEP/pplx for MoE exchange (batchgen/worker/rank_sync_engine.py:595); here one heap serves
every fused collective.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

MAX_WORLD = 8


class SymmetricHeap:
    GUARD_BYTE = 0xA5

    def __init__(self, nbytes: int, device, group=None, guard_bytes: int = 0):
        """``guard_bytes`` > 0 (debug: ``BG_COMM_GUARD=1`` in ``FusedComm``) puts a poisoned band after every region;
        ``check_guards`` then names the regions past whose end somebody - this rank or a peer - has written."""
        import torch.distributed._symmetric_memory as symm_mem
        self.guard_bytes = int(guard_bytes)
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > MAX_WORLD:
            raise ValueError("the fused kernels address at most 8 peers (one NVSwitch domain)")
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.base_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        # multicast (NVLS) address of the same allocation: one store to it reaches every rank's copy; 0 = no support
        try:
            self.mc_base = int(self.handle.multicast_ptr or 0) if self.handle.has_multicast_support else 0
        except (AttributeError, RuntimeError):
            self.mc_base = 0
        assert self.base_ptrs[self.rank] == self.local.data_ptr()
        self._off = 0
        self.regions: Dict[str, Tuple[int, int]] = {}
        torch.cuda.synchronize()
        self.barrier()

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def alloc(self, name: str, nbytes: int, align: int = 1024) -> int:
        off = (self._off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: {name} needs {nbytes} B at {off} of {self.nbytes}")
        self._off = off + nbytes
        self.regions[name] = (off, nbytes)
        if self.guard_bytes:
            g0 = self._off
            if g0 + self.guard_bytes > self.nbytes:
                raise MemoryError(f"symmetric heap exhausted by the guard band of {name}")
            self.local[g0: g0 + self.guard_bytes].fill_(self.GUARD_BYTE)
            self._off = g0 + self.guard_bytes
        return off

    def check_guards(self) -> List[str]:
        """Regions whose guard band no longer holds the poison pattern (call after a synchronisation)."""
        bad = []
        if not self.guard_bytes:
            return bad
        torch.cuda.synchronize()
        for name, (off, nbytes) in self.regions.items():
            band = self.local[off + nbytes: off + nbytes + self.guard_bytes]
            if not bool((band == self.GUARD_BYTE).all()):
                bad.append(name)
        return bad

    def view(self, name: str, dtype: torch.dtype, shape) -> torch.Tensor:
        off, nbytes = self.regions[name]
        t = self.local[off: off + nbytes].view(dtype)
        n = 1
        for s in shape:
            n *= s
        return t[:n].view(*shape)

    def mc_ptr(self, name: str, extra_offset: int = 0) -> int:
        """Multicast address of a region (0 when the allocation has no multicast mapping)."""
        off, _ = self.regions[name]
        return self.mc_base + off + extra_offset if self.mc_base else 0

    def peer_ptrs(self, name: str, extra_offset: int = 0):
        """ctypes array of 8 ``void*``: the region's address on every rank (null past ``world``)."""
        off, _ = self.regions[name]
        arr = (ctypes.c_void_p * MAX_WORLD)()
        for r in range(MAX_WORLD):
            arr[r] = (self.base_ptrs[r] + off + extra_offset) if r < self.world else None
        return arr
