"""IntakePool and SchedulingPool: the two queues between the HTTP front end and the workers.

``IntakePool`` holds tokenised requests that have been accepted but not yet handed to the workers.  It is
capacity limited, has HIGH and NORMAL lanes, and accepts a batch all-or-nothing (a batch that does not fit
is refused whole, so a client never sees half a batch admitted).  ``SchedulingPool`` owns a fixed number
of *slots* — one per request the workers may hold at a time (the worker side reserves the same number of
token-book entries) — and a ``BatchTracker`` per batch that de-duplicates results per (batch, request),
so a result delivered twice (worker restart replay) is counted once.

Reference parity: batchgen/server/intake_pool.py:25-204 (``IntakePool`` :50, ``submit_batch`` :74,
``drain`` :120) and batchgen/server/scheduling_pool.py:23-285 (``SchedulingPool`` :47, ``allocate_slot``
:102, ``record_request_result`` :172).
"""
from __future__ import annotations

import threading
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Set, Tuple

HIGH, NORMAL = 1, 0


@dataclass
class IntakeRequest:
    batch_id: str
    request_id: str            # custom_id within the batch
    prompt_ids: List[int]
    sampling: Dict[str, Any]
    priority: int = NORMAL
    meta: Dict[str, Any] = field(default_factory=dict)


class IntakeFull(RuntimeError):
    pass


class IntakePool:
    def __init__(self, capacity: int):
        self.capacity = capacity
        self._lanes: Dict[int, Deque[IntakeRequest]] = {HIGH: deque(), NORMAL: deque()}
        self._lock = threading.Lock()
        self._cancelled: Set[str] = set()

    def __len__(self) -> int:
        return len(self._lanes[HIGH]) + len(self._lanes[NORMAL])

    @property
    def fill_fraction(self) -> float:
        return len(self) / self.capacity

    def submit_batch(self, reqs: List[IntakeRequest]) -> None:
        """All-or-nothing."""
        with self._lock:
            if len(self) + len(reqs) > self.capacity:
                raise IntakeFull(f"intake holds {len(self)} of {self.capacity}; the batch has {len(reqs)} requests")
            for r in reqs:
                self._lanes[HIGH if r.priority == HIGH else NORMAL].append(r)

    def drain(self, max_items: int) -> List[IntakeRequest]:
        """Up to ``max_items`` requests, HIGH lane first, FIFO inside a lane; cancelled batches are dropped."""
        out: List[IntakeRequest] = []
        with self._lock:
            for lane in (HIGH, NORMAL):
                q = self._lanes[lane]
                while q and len(out) < max_items:
                    r = q.popleft()
                    if r.batch_id in self._cancelled:
                        continue
                    out.append(r)
        return out

    def cancel_batch(self, batch_id: str) -> int:
        with self._lock:
            self._cancelled.add(batch_id)
            n = 0
            for lane in (HIGH, NORMAL):
                keep = deque(r for r in self._lanes[lane] if r.batch_id != batch_id)
                n += len(self._lanes[lane]) - len(keep)
                self._lanes[lane] = keep
            return n


@dataclass
class BatchTracker:
    batch_id: str
    total: int
    done: Set[str] = field(default_factory=set)
    completed: int = 0
    failed: int = 0
    cancelled: bool = False

    @property
    def finished(self) -> bool:
        return len(self.done) >= self.total


class SchedulingPool:
    def __init__(self, slots: int):
        self.slots = slots
        self._free: List[int] = list(range(slots - 1, -1, -1))
        self._by_slot: Dict[int, IntakeRequest] = {}
        self._slot_of: Dict[Tuple[str, str], int] = {}
        self.trackers: Dict[str, BatchTracker] = {}
        self._lock = threading.Lock()

    @property
    def used(self) -> int:
        return self.slots - len(self._free)

    @property
    def free(self) -> int:
        return len(self._free)

    def register_batch(self, batch_id: str, total: int) -> BatchTracker:
        with self._lock:
            t = BatchTracker(batch_id, total)
            self.trackers[batch_id] = t
            return t

    def allocate_slot(self, req: IntakeRequest) -> Optional[int]:
        with self._lock:
            if not self._free:
                return None
            s = self._free.pop()
            self._by_slot[s] = req
            self._slot_of[(req.batch_id, req.request_id)] = s
            return s

    def select_from_intake(self, intake: IntakePool) -> List[Tuple[int, IntakeRequest]]:
        """Move as many requests as there are free slots from the intake pool into slots."""
        out = []
        for r in intake.drain(self.free):
            s = self.allocate_slot(r)
            assert s is not None
            out.append((s, r))
        return out

    def record_request_result(self, batch_id: str, request_id: str, ok: bool) -> Tuple[bool, bool]:
        """-> (counted, batch_finished).  A second result for the same request is ignored."""
        with self._lock:
            t = self.trackers.get(batch_id)
            if t is None or request_id in t.done:
                return False, bool(t and t.finished)
            t.done.add(request_id)
            if ok:
                t.completed += 1
            else:
                t.failed += 1
            s = self._slot_of.pop((batch_id, request_id), None)
            if s is not None:
                self._by_slot.pop(s, None)
                self._free.append(s)
            return True, t.finished

    def in_flight(self, batch_id: Optional[str] = None) -> List[IntakeRequest]:
        with self._lock:
            return [r for r in self._by_slot.values() if batch_id is None or r.batch_id == batch_id]

    def release_batch(self, batch_id: str) -> int:
        """Free every slot still held by a batch (cancel / worker loss)."""
        with self._lock:
            n = 0
            for key in [k for k in self._slot_of if k[0] == batch_id]:
                s = self._slot_of.pop(key)
                self._by_slot.pop(s, None)
                self._free.append(s)
                n += 1
            return n
