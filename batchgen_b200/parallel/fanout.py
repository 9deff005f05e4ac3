"""Streamed-expert fan-out over NVLink (F5): a weight frame that one rank of a replica group brought onto its GPU
is written into the same ring slot of the other members by one kernel, so the frame crosses PCIe once per group.

``ReplicaFanout`` owns a symmetric region of ``slots`` x ``slot_bytes`` (every rank's ring slots at the same offsets,
mapped into every peer) and a flag per (slot, source rank).  The owner calls ``push(slot, members)`` after its
host -> device copy into ``slot_view(slot)``; a member calls ``wait(slot, owner)`` (a bounded device-side wait on the
compute stream) before its expert GEMM reads the slot.  With NVLS (``BG_NVLS=1`` and a multicast mapping) a frame is
broadcast with ``multimem.st``; otherwise the kernel stores to each member in turn.

Which rank owns which frame, and when a slot may be overwritten, is the business of ``core.weight_replica``
(ownership + frame plan) and of the replica control block (``core.native.ReplicaControlBlock``: publish / ack);
this class is the data path only.

Reference parity: core/HtoD_Engine/HtoD_Engine.cu:1395-1434 (peer fan-out of a streamed expert),
core/GPU_Weight_Buffer/GPU_Weight_Buffer.h:53-245 (peer-visible ring slots).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _ext
from .symm import SymmetricHeap


class ReplicaFanout:
    def __init__(self, slots: int, slot_bytes: int, device, group=None):
        if slot_bytes % 16:
            raise ValueError("slot_bytes must be a multiple of 16")
        self.device = torch.device(device)
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.slots, self.slot_bytes = slots, slot_bytes
        flags_bytes = slots * self.world * 4
        self.heap = SymmetricHeap(slots * slot_bytes + flags_bytes + 2 * 1024 + 64 * 1024, self.device, self.group)
        self.heap.alloc("flags", flags_bytes)
        self.heap.alloc("ring", slots * slot_bytes)
        self.ring = self.heap.view("ring", torch.uint8, (slots, slot_bytes))
        self.flags = self.heap.view("flags", torch.int32, (slots * self.world,))
        self.flag_ptrs = self.heap.peer_ptrs("flags")
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = _ext.status_word(self.device)
        self.epoch = [0] * slots                       # per slot: number of frames published into it so far
        self.nvls = os.environ.get("BG_NVLS", "0") == "1" and self.heap.mc_base != 0
        self.heap.barrier()

    def slot_view(self, slot: int) -> torch.Tensor:
        """This rank's copy of a ring slot (uint8 [slot_bytes]): the owner fills it, members read it."""
        return self.ring[slot]

    def push(self, slot: int, members, nbytes: int = 0) -> None:
        """Owner side: copy ``nbytes`` (default: the whole slot) of this rank's slot into the slot of every rank in
        ``members`` and raise their arrival flag.  Every rank of the group must call ``advance(slot)`` or ``push`` /
        ``wait`` once per frame so that the per-slot epochs stay in step."""
        nbytes = nbytes or self.slot_bytes
        if nbytes % 16 or nbytes > self.slot_bytes:
            raise ValueError("frame size must be a multiple of 16 bytes within the slot")
        mask = 0
        for r in members:
            if r != self.rank:
                mask |= 1 << int(r)
        self.epoch[slot] += 1
        if mask == 0:
            return
        off = slot * self.slot_bytes
        mc = self.heap.mc_ptr("ring", off) if self.nvls else 0
        rc = _ext.lib().bg_fanout_push(
            ctypes.c_void_p(self.ring[slot].data_ptr()), self.heap.peer_ptrs("ring", off),
            ctypes.c_ulonglong(nbytes), ctypes.c_uint(mask), ctypes.c_void_p(mc), ctypes.c_int(self.rank),
            ctypes.c_int(self.world), self.flag_ptrs, ctypes.c_int(slot * self.world), ctypes.c_uint32(self.epoch[slot]),
            ctypes.c_void_p(0), _ext.ptr(self.counter), ctypes.c_int(_ext.num_sms(self.device)), _ext.stream())
        _ext.check(rc, "bg_fanout_push")

    def wait(self, slot: int, owner: int) -> None:
        """Member side: the compute stream waits (bounded, on the device) until ``owner``'s frame for this slot's
        next epoch has landed."""
        self.epoch[slot] += 1
        flag = ctypes.c_void_p(self.flags.data_ptr() + 4 * (slot * self.world + owner))
        rc = _ext.lib().bg_wait_flags(flag, ctypes.c_int(1), ctypes.c_uint32(self.epoch[slot]), ctypes.c_void_p(0),
                                      _ext.ptr(self.status), _ext.stream())
        _ext.check(rc, "bg_wait_flags")

    def advance(self, slot: int) -> None:
        """A rank that neither sends nor receives this frame keeps its epoch counter in step."""
        self.epoch[slot] += 1
