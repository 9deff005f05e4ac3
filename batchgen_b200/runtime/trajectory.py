"""Trajectory frontiers: cross-wave KV reuse for agent sessions (one session = one trajectory of turns).

When a turn finishes, the engine may *commit* the session's KV up to a page-aligned boundary (the frontier):
the latent-KV host pages plus, for models with recurrent layers, ONE state snapshot taken at the same
boundary.  The two halves form one record with one refcount, so a hit can never find pages without a
snapshot or the reverse.  The next turn of the session, whose prompt extends the committed tokens, restores
the record (its pages are loaded, nothing is recomputed) and prefill starts at the boundary.

* the hit predicate is binary: the longest common prefix of the new prompt and the committed tokens must
  cover the whole frontier (a partial match restores nothing);
* a session owns at most one record: ``advance`` replaces it (the old one leaves when its last reader drops it);
* every refusal is named (``DECLINE_*``); nothing degrades silently;
* the registry reports what it holds (pages, snapshot bytes) so admission can charge it.

Pure host bookkeeping: the device->host copy, page retention and admission wiring are done by the caller
through the ``release_fn`` callback.

Reference parity: batchgen/prefix_reuse/trajectory_frontier.py:337-411 (session key, index key, hit
predicate), :438-510 (charge), :522-745 (record, acquire/release), :774-1100 (registry: resolve, begin,
advance, evict, invariants); trajectory_commit.py / trajectory_restore.py (commit after a turn, restore at
admission, named decline reasons).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

DECLINE_NO_SESSION = "no_committed_frontier_for_session"
DECLINE_PROMPT_DIVERGES = "prompt_does_not_extend_frontier"
DECLINE_PROMPT_TOO_SHORT = "prompt_leaves_no_private_token_after_frontier"
DECLINE_NAMESPACE = "model_or_layout_namespace_changed"
DECLINE_RELEASED = "frontier_already_released"


class TrajectoryFrontierError(RuntimeError):
    pass


class FrontierRefcountError(TrajectoryFrontierError):
    pass


class FrontierRegistryError(TrajectoryFrontierError):
    pass


def aligned_prefix_tokens(n_tokens: int, page_tokens: int) -> int:
    """Largest page-aligned prefix that still leaves the last token private."""
    return max(0, (n_tokens - 1) // page_tokens) * page_tokens


def session_key_for(session_id: str, namespace: Sequence[int] = ()) -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(session_id.encode())
    for v in namespace:
        h.update(int(v).to_bytes(8, "little", signed=True))
    return h.hexdigest()


def longest_common_prefix_length(a: Sequence[int], b: Sequence[int]) -> int:
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return n


def is_frontier_hit(*, lcp_tokens: int, frontier_boundary_tokens: int) -> bool:
    return frontier_boundary_tokens > 0 and lcp_tokens >= frontier_boundary_tokens


@dataclass(frozen=True)
class StateSnapshot:
    """Recurrent-state snapshot taken at the frontier boundary (e.g. linear-attention state + conv tails):
    where it lives in the host arena and how large it is.  ``None`` on the record for pure-MLA models."""
    arena_offset: int
    nbytes: int
    shards: int = 1


@dataclass(frozen=True)
class FrontierCharge:
    pages: int
    page_bytes: int
    snapshot_bytes: int

    @property
    def total_bytes(self) -> int:
        return self.pages * self.page_bytes + self.snapshot_bytes


class TrajectoryFrontierRecord:
    def __init__(self, session_key: str, namespace: Tuple[int, ...], token_ids: Sequence[int], page_tokens: int,
                 page_ids: Sequence[int], page_bytes: int, snapshot: Optional[StateSnapshot], owning_group: int,
                 release_fn: Callable[["TrajectoryFrontierRecord"], None]):
        if len(token_ids) == 0 or len(token_ids) % page_tokens:
            raise TrajectoryFrontierError("a frontier must be a non-empty whole number of pages")
        if len(page_ids) != len(token_ids) // page_tokens:
            raise TrajectoryFrontierError("one host page per page of frontier tokens")
        self.session_key, self.namespace = session_key, tuple(namespace)
        self.token_ids = tuple(int(t) for t in token_ids)
        self.page_tokens, self.page_ids, self.page_bytes = page_tokens, tuple(page_ids), page_bytes
        self.snapshot, self.owning_group = snapshot, owning_group
        self._release_fn = release_fn
        self._refs = 1                     # the registry's own reference
        self._released = False

    @property
    def boundary_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def refcount(self) -> int:
        return self._refs

    @property
    def is_released(self) -> bool:
        return self._released

    @property
    def charge(self) -> FrontierCharge:
        return FrontierCharge(len(self.page_ids), self.page_bytes, self.snapshot.nbytes * self.snapshot.shards
                              if self.snapshot else 0)

    def acquire(self) -> "TrajectoryFrontierRecord":
        if self._released or self._refs <= 0:
            raise FrontierRefcountError("acquire on a released frontier")
        self._refs += 1
        return self

    def release(self) -> bool:
        """Drop one reference; pages and snapshot leave together with the last one.  True if released."""
        if self._refs <= 0:
            raise FrontierRefcountError("release without a reference")
        self._refs -= 1
        if self._refs == 0 and not self._released:
            self._released = True
            self._release_fn(self)
            return True
        return False


@dataclass(frozen=True)
class FrontierResolution:
    hit: bool
    reason: Optional[str]
    record: Optional[TrajectoryFrontierRecord] = None

    @property
    def boundary_tokens(self) -> int:
        return self.record.boundary_tokens if self.hit else 0


class TrajectoryFrontierRegistry:
    def __init__(self, page_tokens: int, page_bytes: int, namespace: Sequence[int] = (),
                 release_fn: Optional[Callable[[TrajectoryFrontierRecord], None]] = None):
        self.page_tokens, self.page_bytes, self.namespace = page_tokens, page_bytes, tuple(namespace)
        self._release_fn = release_fn or (lambda rec: None)
        self._records: Dict[str, TrajectoryFrontierRecord] = {}
        self.stats = {"commits": 0, "hits": 0, "declines": 0, "evictions": 0}

    def __len__(self) -> int:
        return len(self._records)

    def key(self, session_id: str) -> str:
        return session_key_for(session_id, self.namespace)

    def get(self, session_id: str) -> Optional[TrajectoryFrontierRecord]:
        return self._records.get(self.key(session_id))

    # ------------------------------------------------------------------ commit
    def advance(self, session_id: str, token_ids: Sequence[int], page_ids: Sequence[int],
                snapshot: Optional[StateSnapshot] = None, owning_group: int = 0) -> TrajectoryFrontierRecord:
        """Commit the trajectory up to the aligned boundary of ``token_ids`` (all tokens of the finished
        turn, prompt + generated); ``page_ids`` are the host pages of that prefix.  Replaces the session's
        previous frontier, which leaves when its last reader drops it."""
        boundary = aligned_prefix_tokens(len(token_ids), self.page_tokens)
        if boundary == 0:
            raise FrontierRegistryError("trajectory shorter than one page: nothing to commit")
        n_pages = boundary // self.page_tokens
        if len(page_ids) < n_pages:
            raise FrontierRegistryError(f"{n_pages} pages needed, {len(page_ids)} given")
        k = self.key(session_id)
        rec = TrajectoryFrontierRecord(k, self.namespace, token_ids[:boundary], self.page_tokens, page_ids[:n_pages],
                                       self.page_bytes, snapshot, owning_group, self._release_fn)
        old = self._records.get(k)
        self._records[k] = rec
        if old is not None:
            old.release()
        self.stats["commits"] += 1
        return rec

    # ------------------------------------------------------------------ restore
    def resolve(self, session_id: str, prompt_ids: Sequence[int], namespace: Optional[Sequence[int]] = None
                ) -> FrontierResolution:
        """Can the next turn's prompt restore the session's frontier?  A hit takes a reference that the
        caller drops (``record.release()``) once the pages are loaded or the restore is abandoned."""
        def decline(reason):
            self.stats["declines"] += 1
            return FrontierResolution(False, reason)

        if namespace is not None and tuple(namespace) != self.namespace:
            return decline(DECLINE_NAMESPACE)
        rec = self._records.get(self.key(session_id))
        if rec is None:
            return decline(DECLINE_NO_SESSION)
        if rec.is_released:
            return decline(DECLINE_RELEASED)
        if len(prompt_ids) <= rec.boundary_tokens:
            return decline(DECLINE_PROMPT_TOO_SHORT)
        lcp = longest_common_prefix_length(prompt_ids, rec.token_ids)
        if not is_frontier_hit(lcp_tokens=lcp, frontier_boundary_tokens=rec.boundary_tokens):
            return decline(DECLINE_PROMPT_DIVERGES)
        self.stats["hits"] += 1
        return FrontierResolution(True, None, rec.acquire())

    # ------------------------------------------------------------------ eviction / accounting
    def evict(self, session_id: str) -> bool:
        rec = self._records.pop(self.key(session_id), None)
        if rec is None:
            raise FrontierRegistryError(f"session {session_id!r} holds no frontier")
        self.stats["evictions"] += 1
        return rec.release()

    def evict_for_pages(self, want_pages: int, lru_order: Iterable[str]) -> int:
        """Evict unread frontiers in the given order until ``want_pages`` host pages are back."""
        freed = 0
        for sid in list(lru_order):
            if freed >= want_pages:
                break
            rec = self.get(sid)
            if rec is not None and rec.refcount == 1:
                freed += len(rec.page_ids)
                self.evict(sid)
        return freed

    def total_charge(self) -> FrontierCharge:
        pages = sum(len(r.page_ids) for r in self._records.values())
        snap = sum(r.charge.snapshot_bytes for r in self._records.values())
        return FrontierCharge(pages, self.page_bytes, snap)

    def session_group_summary(self) -> Dict[str, Tuple[int, int]]:
        """session key -> (owning decode group, boundary tokens): lets admission pin the next turn to the
        group whose node holds the pages."""
        return {k: (r.owning_group, r.boundary_tokens) for k, r in self._records.items()}

    def check_invariants(self) -> None:
        for k, r in self._records.items():
            if r.session_key != k or r.is_released or r.refcount < 1:
                raise TrajectoryFrontierError(f"registry holds a dead or misfiled record for {k}")
            if r.boundary_tokens % self.page_tokens or len(r.page_ids) * self.page_tokens != r.boundary_tokens:
                raise TrajectoryFrontierError(f"record {k} is not page aligned")
