"""Named start-up phases that the server's watchdog can read while a worker is stuck.

A cold start is a chain of long, silent steps (checkpoint staging, communicator rendezvous, model build, KV pool,
graph capture).  One that never returns looks from outside like one that is slow.  Every process of a start-up
writes the phase it is in and the time it entered it into its own slot of a shared, lock-free record; the manager
polls the record and, when a slot has stayed in one phase longer than that phase's budget, fails the start-up with
the slot, the phase and the seconds in its message.  The budget restarts at every phase entry: a start-up that is
slow but moving is never killed for its total time (that is what ``--startup-timeout`` is for).

The record is a raw shared array (no lock that a stuck or dead writer could hold).  Each slot has one writer; a
per-slot sequence number, odd while a write is in progress, lets the reader skip a half-written slot.
``time.monotonic`` is system-wide on Linux, so a time written by a worker compares with the manager's clock.

Reference parity: batchgen/worker/startup_phases.py:1-60 (shared phase record, per-entry budgets, named stalls).
"""
from __future__ import annotations

import contextlib
import multiprocessing as mp
import time
from typing import Dict, Iterator, List, Optional, Tuple

PHASES: Tuple[str, ...] = ("spawned", "store-staging", "communicator-init", "model-build", "kv-pool",
                           "graph-capture", "prewarm", "serving")
_INDEX = {n: i for i, n in enumerate(PHASES)}

# generous: the watchdog ends start-ups that hang, not ones that are slow
DEFAULT_BUDGETS: Dict[str, float] = {"spawned": 300.0, "store-staging": 3600.0, "communicator-init": 600.0,
                                     "model-build": 3600.0, "kv-pool": 600.0, "graph-capture": 1800.0,
                                     "prewarm": 900.0}
_FIELDS = 3     # sequence number, phase index, time of entry


class StartupRecord:
    def __init__(self, slots: int, ctx=None):
        self.slots = slots
        self._a = (ctx or mp.get_context("spawn")).RawArray("d", slots * _FIELDS)
        for s in range(slots):
            self._a[s * _FIELDS + 1] = -1.0

    # ---- writer side (one process per slot)
    def enter(self, slot: int, phase: str) -> None:
        b = slot * _FIELDS
        seq = self._a[b]
        self._a[b] = seq + 1                      # odd: write in progress
        self._a[b + 1] = float(_INDEX[phase])
        self._a[b + 2] = time.monotonic()
        self._a[b] = seq + 2

    @contextlib.contextmanager
    def phase(self, slot: int, name: str) -> Iterator[None]:
        self.enter(slot, name)
        yield

    # ---- reader side
    def read(self, slot: int) -> Optional[Tuple[str, float]]:
        """(phase, time of entry) of a slot, or None if it has not started or a write is in progress."""
        b = slot * _FIELDS
        for _ in range(4):
            s0 = self._a[b]
            idx, t = self._a[b + 1], self._a[b + 2]
            if s0 == self._a[b] and int(s0) % 2 == 0:
                return (PHASES[int(idx)], t) if idx >= 0 else None
        return None

    def stalled(self, budgets: Optional[Dict[str, float]] = None, now: Optional[float] = None
                ) -> List[Tuple[int, str, float, float]]:
        """Slots that have sat in one phase past its budget: (slot, phase, seconds in it, budget)."""
        budgets = DEFAULT_BUDGETS if budgets is None else budgets
        now = time.monotonic() if now is None else now
        out = []
        for s in range(self.slots):
            r = self.read(s)
            if r is None:
                continue
            phase, t = r
            limit = budgets.get(phase)
            if limit is not None and now - t > limit:
                out.append((s, phase, now - t, limit))
        return out

    def snapshot(self) -> Dict[int, Tuple[str, float]]:
        now = time.monotonic()
        return {s: (r[0], now - r[1]) for s in range(self.slots) if (r := self.read(s)) is not None}


class _NullRecord:
    """Stands in when a worker runs without a manager (in-process tests)."""

    def enter(self, slot: int, phase: str) -> None:
        pass

    @contextlib.contextmanager
    def phase(self, slot: int, name: str) -> Iterator[None]:
        yield


def record_of(args) -> "StartupRecord":
    return getattr(args, "startup_record", None) or _NullRecord()
