"""QueryBook: a fixed-byte-budget paged book of token ids (prompt + generated) for every live sequence.

One int32 CPU tensor of pages holds all trajectories.  ``bind`` reserves, up front, every page a sequence
can ever need (prompt + maximum generated suffix) as ONE contiguous extent, so a request either gets its
full reservation or stays queued, and appending a token is an index increment on a cached tail (no page
table lookup on the hot path).  Free space is kept as extents, so allocator metadata is proportional to
fragmentation and not to the byte budget.  A trajectory is a list of *turns* (agent sessions re-enter with a
longer prompt); each turn records its prompt end and generated end.

The storage can live in an anonymous memfd shared by all workers of a node (``NodeSharedTokens``): prompt
ids are identical on every rank, so one copy per node replaces one per rank.

Reference parity: batchgen/query_book.py:61-1190 (book, bind/release, turns, append, restore, copy);
batchgen/batchgen_worker.py:596-740 (node-shared memfd and tensor allocation).
"""
from __future__ import annotations

import mmap
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class QueryBookTurn:
    token_start: int
    prompt_end: int
    generated_end: int


@dataclass
class QueryBookSlot:
    slot: int
    sequence_id: str
    max_tokens: int
    length: int = 0                 # tokens written so far (prompt + generated, all turns)

    @property
    def remaining(self) -> int:
        return self.max_tokens - self.length


class QueryBook:
    TOKEN_BYTES = 4

    def __init__(self, capacity_bytes: int, page_tokens: int = 4096, storage: Optional[torch.Tensor] = None):
        if capacity_bytes <= 0 or page_tokens <= 0:
            raise ValueError("capacity_bytes and page_tokens must be positive")
        self.page_tokens = int(page_tokens)
        self.page_bytes = self.page_tokens * self.TOKEN_BYTES
        if capacity_bytes < self.page_bytes:
            raise ValueError(f"capacity_bytes={capacity_bytes} is smaller than one page={self.page_bytes}")
        self.page_count = capacity_bytes // self.page_bytes
        if storage is None:
            storage = torch.empty((self.page_count, self.page_tokens), dtype=torch.int32)
        if storage.dtype != torch.int32 or storage.device.type != "cpu" or not storage.is_contiguous() \
                or tuple(storage.shape) != (self.page_count, self.page_tokens):
            raise ValueError(f"storage must be a contiguous CPU int32 tensor of shape ({self.page_count}, {self.page_tokens})")
        self.storage = storage
        self._flat = storage.view(-1)
        self._free: List[Tuple[int, int]] = [(0, self.page_count)]     # (first page, pages), sorted by start
        self._slots: Dict[int, QueryBookSlot] = {}
        self._range: Dict[int, Tuple[int, int]] = {}
        self._turns: Dict[int, List[QueryBookTurn]] = {}
        self._by_seq: Dict[str, int] = {}
        self._free_slots: List[int] = []
        self._next_slot = 0

    # ------------------------------------------------------------------ capacity
    @property
    def free_page_count(self) -> int:
        return sum(n for _, n in self._free)

    @property
    def largest_free_extent_pages(self) -> int:
        return max((n for _, n in self._free), default=0)

    @property
    def active_count(self) -> int:
        return len(self._slots)

    def pages_for(self, max_tokens: int) -> int:
        return max(1, -(-int(max_tokens) // self.page_tokens))

    def can_reserve(self, max_tokens: int) -> bool:
        return self.largest_free_extent_pages >= self.pages_for(max_tokens)

    def can_reserve_batch(self, max_tokens: Sequence[int]) -> bool:
        """First-fit of the whole batch (largest first) into a copy of the free list."""
        free = list(self._free)
        for need in sorted((self.pages_for(t) for t in max_tokens), reverse=True):
            for i, (s, n) in enumerate(free):
                if n >= need:
                    free[i] = (s + need, n - need)
                    break
            else:
                return False
        return True

    # ------------------------------------------------------------------ bind / release
    def _take(self, pages: int) -> int:
        for i, (s, n) in enumerate(self._free):
            if n >= pages:
                if n == pages:
                    self._free.pop(i)
                else:
                    self._free[i] = (s + pages, n - pages)
                return s
        raise MemoryError(f"no free extent of {pages} pages (largest {self.largest_free_extent_pages})")

    def _give(self, start: int, pages: int) -> None:
        self._free.append((start, pages))
        self._free.sort()
        merged: List[Tuple[int, int]] = []
        for s, n in self._free:
            if merged and merged[-1][0] + merged[-1][1] == s:
                merged[-1] = (merged[-1][0], merged[-1][1] + n)
            else:
                merged.append((s, n))
        self._free = merged

    def bind(self, sequence_id: str, max_tokens: int) -> int:
        if sequence_id in self._by_seq:
            raise ValueError(f"sequence {sequence_id!r} is already bound")
        pages = self.pages_for(max_tokens)
        start = self._take(pages)
        slot = self._free_slots.pop() if self._free_slots else self._next_slot
        if slot == self._next_slot:
            self._next_slot += 1
        self._slots[slot] = QueryBookSlot(slot, sequence_id, int(max_tokens))
        self._range[slot] = (start, pages)
        self._turns[slot] = []
        self._by_seq[sequence_id] = slot
        return slot

    def bind_batch(self, sequence_ids: Sequence[str], max_tokens: Sequence[int]) -> List[int]:
        """All or nothing."""
        if not self.can_reserve_batch(max_tokens):
            raise MemoryError("the batch does not fit the token book")
        order = sorted(range(len(sequence_ids)), key=lambda i: -self.pages_for(max_tokens[i]))
        slots = [0] * len(sequence_ids)
        for i in order:
            slots[i] = self.bind(sequence_ids[i], max_tokens[i])
        return slots

    def release(self, slot: int) -> None:
        meta = self._slots.pop(slot)
        self._give(*self._range.pop(slot))
        self._turns.pop(slot)
        del self._by_seq[meta.sequence_id]
        self._free_slots.append(slot)

    def slot_for(self, sequence_id: str) -> int:
        return self._by_seq[sequence_id]

    def has_sequence(self, sequence_id: str) -> bool:
        return sequence_id in self._by_seq

    def metadata(self, slot: int) -> QueryBookSlot:
        return self._slots[slot]

    def turns(self, slot: int) -> Tuple[QueryBookTurn, ...]:
        return tuple(self._turns[slot])

    # ------------------------------------------------------------------ writing
    def _base(self, slot: int) -> int:
        return self._range[slot][0] * self.page_tokens

    def _write(self, slot: int, tokens: torch.Tensor) -> Tuple[int, int]:
        meta = self._slots[slot]
        t = tokens.to(torch.int32).reshape(-1)
        if t.numel() > meta.remaining:
            raise ValueError(f"slot {slot}: {t.numel()} tokens exceed the reservation ({meta.remaining} left)")
        a = self._base(slot) + meta.length
        self._flat[a:a + t.numel()] = t
        start = meta.length
        meta.length += t.numel()
        return start, meta.length

    def write_prompt(self, slot: int, prompt_tokens: torch.Tensor) -> QueryBookTurn:
        """First turn: the prompt of a freshly bound sequence."""
        if self._slots[slot].length or self._turns[slot]:
            raise ValueError(f"slot {slot} already holds tokens; use append_prompt for a new turn")
        return self.append_prompt(slot, prompt_tokens)

    def append_prompt(self, slot: int, prompt_tokens: torch.Tensor) -> QueryBookTurn:
        """A new turn: further prompt tokens after everything written so far."""
        start, end = self._write(slot, prompt_tokens)
        turn = QueryBookTurn(start, end, end)
        self._turns[slot].append(turn)
        return turn

    def begin_reentry_turn(self, slot: int, prompt_length: int) -> QueryBookTurn:
        """An evicted sequence re-enters with everything written so far as its prompt: the generated tokens of
        earlier turns become prompt tokens of the new turn (recompute), nothing is copied."""
        meta = self._slots[slot]
        if prompt_length != meta.length:
            raise ValueError(f"slot {slot}: re-entry prompt length {prompt_length} != tokens held {meta.length}")
        turn = QueryBookTurn(0, meta.length, meta.length)
        self._turns[slot].append(turn)
        return turn

    def append_token(self, slot: int, token_id: int) -> int:
        meta = self._slots[slot]
        if meta.remaining <= 0:
            raise ValueError(f"slot {slot} is full ({meta.max_tokens} tokens)")
        if not self._turns[slot]:
            raise ValueError(f"slot {slot} has no open turn")
        self._flat[self._base(slot) + meta.length] = int(token_id)
        meta.length += 1
        self._turns[slot][-1].generated_end = meta.length
        return meta.length

    def append_tokens(self, slots: Sequence[int], token_ids: Sequence[int]) -> None:
        for s, t in zip(slots, token_ids):
            self.append_token(s, t)

    # ------------------------------------------------------------------ reading
    def tokens(self, slot: int, length: Optional[int] = None) -> torch.Tensor:
        meta = self._slots[slot]
        n = meta.length if length is None else int(length)
        if not 0 <= n <= meta.length:
            raise ValueError(f"slot {slot}: length {n} outside [0, {meta.length}]")
        a = self._base(slot)
        return self._flat[a:a + n]

    def generated_tokens(self, slot: int) -> torch.Tensor:
        """Generated tokens of the current turn."""
        turn = self._turns[slot][-1]
        a = self._base(slot)
        return self._flat[a + turn.prompt_end:a + turn.generated_end]

    def last_generated_token(self, slot: int) -> int:
        g = self.generated_tokens(slot)
        if g.numel() == 0:
            raise ValueError(f"slot {slot} has generated nothing in this turn")
        return int(g[-1])

    def copy_to(self, slot: int, other: "QueryBook", other_slot: int) -> None:
        """Copy a trajectory (tokens and turns) into a bound, empty slot of another book (migration)."""
        if other._slots[other_slot].length:
            raise ValueError("destination slot is not empty")
        other._write(other_slot, self.tokens(slot))
        other._turns[other_slot] = [QueryBookTurn(t.token_start, t.prompt_end, t.generated_end) for t in self._turns[slot]]

    def audit(self) -> int:
        """Number of broken invariants (overlapping extents, lengths beyond reservations)."""
        bad = 0
        spans = sorted(list(self._free) + list(self._range.values()))
        pos = 0
        for s, n in spans:
            bad += s != pos
            pos = s + n
        bad += pos != self.page_count
        for slot, meta in self._slots.items():
            bad += meta.length > self._range[slot][1] * self.page_tokens or meta.length > meta.max_tokens
        return bad


class NodeSharedTokens:
    """An anonymous memfd holding one int32 ``[pages, page_tokens]`` table for all workers of a node.  The
    creator makes it; the others attach through ``/proc/<creator pid>/fd/<fd>``.  The region has no name in
    the file system, so the kernel reclaims it with the last mapping however the processes die."""

    def __init__(self, fd: int, mapping: mmap.mmap, rows: int, width: int, creator_pid: int):
        self.fd, self.mapping, self.rows, self.width, self.creator_pid = fd, mapping, rows, width, creator_pid
        self.tensor = torch.frombuffer(mapping, dtype=torch.int32, count=rows * width).view(rows, width)

    @classmethod
    def create(cls, rows: int, width: int) -> "NodeSharedTokens":
        fd = os.memfd_create("bg_query_book")
        os.ftruncate(fd, rows * width * 4)
        return cls(fd, mmap.mmap(fd, rows * width * 4), rows, width, os.getpid())

    def handle(self) -> Tuple[int, int, int, int]:
        """What the creator publishes to the other workers of the node."""
        return (self.creator_pid, self.fd, self.rows, self.width)

    @classmethod
    def attach(cls, handle: Tuple[int, int, int, int]) -> "NodeSharedTokens":
        pid, fd, rows, width = handle
        own = os.open(f"/proc/{pid}/fd/{fd}", os.O_RDWR)
        return cls(own, mmap.mmap(own, rows * width * 4), rows, width, pid)

    def release_fd(self) -> None:
        """Drop the descriptor only: the mapping keeps the region alive while views are in use."""
        if self.fd >= 0:
            try:
                os.close(self.fd)
            except OSError:
                pass
            self.fd = -1
