"""Page-level prefix cache: a tree keyed by a hash chain over page-sized blocks of token ids.

``key(block i) = H(key(block i-1) || tokens of block i)`` (256-bit), so equal keys mean equal
prefixes up to and including that block.  Entries hold one reference on their KV page; a lookup
returns the longest cached chain and the caller shares those pages into a sequence.  Unreferenced
entries (only the cache holds the page) are reclaimable in LRU order, leaves first.

Reference parity: core/KV_Storage/host_prefix_cache_coordinator.h:13-174 (commit /
lookup_and_attach / evict / clear over a 256-bit page hash chain, ``BuildPrefixHashChain`` :101) and
its Python client batchgen/prefix_reuse/prefill.py:64, commit.py:10-30, eviction.py:11-25.  The
native coordinator in ``core/csrc/host_kv.cpp`` (the prefix methods of ``core.native.HostPagedKV``) implements the same contract
for the node-shared host tier; this class is the in-process (per-rank GPU pool) variant and the executable spec.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence as Seq, Tuple

from .kv_cache import PageAllocator


def build_prefix_hash_chain(token_ids: Seq[int], page_size: int, salt: bytes = b"") -> List[bytes]:
    """One 32-byte key per *full* page of ``token_ids``."""
    keys: List[bytes] = []
    prev = hashlib.sha256(b"bg-prefix-root" + salt).digest()
    for i in range(len(token_ids) // page_size):
        blk = token_ids[i * page_size:(i + 1) * page_size]
        prev = hashlib.sha256(prev + struct.pack(f"<{page_size}i", *blk)).digest()
        keys.append(prev)
    return keys


@dataclass
class _Entry:
    page: int
    parent: Optional[bytes]
    children: int = 0


class PrefixCache:
    def __init__(self, allocator: PageAllocator, page_size: int):
        self.alloc, self.page_size = allocator, page_size
        self._entries: "OrderedDict[bytes, _Entry]" = OrderedDict()
        self.hits = self.misses = self.committed = self.evicted = 0

    def __len__(self) -> int:
        return len(self._entries)

    def lookup(self, token_ids: Seq[int], max_tokens: Optional[int] = None) -> Tuple[List[int], List[bytes]]:
        """Longest cached prefix -> (pages, keys).  Never covers the whole prompt: at least one
        token is left to compute so that the last position produces logits."""
        limit = len(token_ids) - 1 if max_tokens is None else min(max_tokens, len(token_ids) - 1)
        keys = build_prefix_hash_chain(token_ids[: max(limit, 0)], self.page_size)
        pages: List[int] = []
        hit: List[bytes] = []
        for k in keys:
            e = self._entries.get(k)
            if e is None:
                break
            self._entries.move_to_end(k)
            pages.append(e.page)
            hit.append(k)
        if pages:
            self.hits += 1
        else:
            self.misses += 1
        return pages, hit

    def page_of(self, key: bytes) -> Optional[int]:
        """The cached page of a chain key, without touching the LRU order or the hit counters."""
        e = self._entries.get(key)
        return None if e is None else e.page

    def attach(self, pages: Seq[int]) -> None:
        """A sequence starts using cached pages: take a reference for it."""
        self.alloc.share(pages)

    def commit(self, token_ids: Seq[int], pages: Seq[int]) -> int:
        """Publish the full pages of a prefilled sequence.  Returns the number of new entries."""
        keys = build_prefix_hash_chain(token_ids, self.page_size)
        new = 0
        parent = None
        for k, p in zip(keys, pages):
            e = self._entries.get(k)
            if e is None:
                self.alloc.share([p])
                self._entries[k] = _Entry(p, parent)
                if parent is not None:
                    self._entries[parent].children += 1
                new += 1
            self._entries.move_to_end(k)
            parent = k
        self.committed += new
        return new

    def reclaimable_pages(self) -> int:
        return sum(1 for e in self._entries.values() if self.alloc.refcount(e.page) == 1)

    def evict(self, want_pages: int, on_evict=None) -> int:
        """Free up to ``want_pages`` pages held only by the cache, LRU leaves first.  ``on_evict(key, page)`` sees
        every page before it goes; when it returns True it has taken over the page's release (a copy that still
        reads the page is in flight) and the page counts as freed."""
        freed = 0
        progress = True
        while freed < want_pages and progress:
            progress = False
            for k in list(self._entries.keys()):
                e = self._entries[k]
                if e.children == 0 and self.alloc.refcount(e.page) == 1:
                    if on_evict is None or not on_evict(k, e.page):
                        self.alloc.free([e.page])
                    if e.parent is not None and e.parent in self._entries:
                        self._entries[e.parent].children -= 1
                    del self._entries[k]
                    freed += 1
                    progress = True
                    if freed >= want_pages:
                        break
        self.evicted += freed
        return freed

    def clear(self) -> int:
        n = 0
        for e in self._entries.values():
            self.alloc.free([e.page])
            n += 1
        self._entries.clear()
        return n

    def stats(self) -> Dict[str, int]:
        return dict(entries=len(self._entries), hits=self.hits, misses=self.misses, committed=self.committed,
                    evicted=self.evicted, reclaimable=self.reclaimable_pages())
