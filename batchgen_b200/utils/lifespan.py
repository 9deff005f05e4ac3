"""Per-sequence lifespan rings: the last N state transitions and KV operations of every live sequence, dumped
when an anomaly is detected (context-length mismatch, repetition, completion without a stop reason).

Off by default (``BG_SEQ_LIFESPAN=1`` turns it on); when off every call is a no-op.

Reference parity: batchgen/lifespan.py:1-200 (SeqEvent, ring buffer, anomaly dump).
"""
from __future__ import annotations

import enum
import json
import os
import time
from collections import deque
from typing import Deque, Dict, List, Optional, Tuple

ENABLED = os.environ.get("BG_SEQ_LIFESPAN", "0") == "1"
MAX_EVENTS = 256
_T0 = time.perf_counter()


class SeqEvent(enum.IntEnum):
    CREATED = 0
    PREFILL_START = 1
    PREFILL_DONE = 2
    DECODE_START = 3
    ON_HOLD = 4
    EVICTED = 5
    REENTRY_START = 6
    COMPLETED = 7
    KV_LOAD_START = 10
    KV_LOAD_DONE = 11
    KV_APPEND = 12
    MIGRATE_SEND = 20
    MIGRATE_RECV = 21
    CTX_REPAIR = 30
    ANOMALY = 40


class LifespanRecorder:
    def __init__(self, enabled: Optional[bool] = None, max_events: int = MAX_EVENTS, dump_dir: Optional[str] = None):
        self.enabled = ENABLED if enabled is None else enabled
        self.max_events, self.dump_dir = max_events, dump_dir
        self._rings: Dict[str, Deque[Tuple[float, int, int, str]]] = {}
        self.dumps: List[str] = []

    def record(self, uuid: str, event: SeqEvent, value: int = 0, note: str = "") -> None:
        if not self.enabled:
            return
        ring = self._rings.get(uuid)
        if ring is None:
            ring = self._rings[uuid] = deque(maxlen=self.max_events)
        ring.append((time.perf_counter() - _T0, int(event), int(value), note))

    def events(self, uuid: str) -> List[Tuple[float, SeqEvent, int, str]]:
        return [(t, SeqEvent(e), v, n) for t, e, v, n in self._rings.get(uuid, ())]

    def forget(self, uuid: str) -> None:
        self._rings.pop(uuid, None)

    def check_context(self, uuid: str, expected_tokens: int, cache_tokens: int) -> bool:
        """True when consistent; a mismatch between the trajectory length and the KV length is an anomaly."""
        if expected_tokens == cache_tokens:
            return True
        self.anomaly(uuid, f"CTX_MISMATCH expected={expected_tokens} cache={cache_tokens}")
        return False

    def check_repetition(self, uuid: str, tokens: List[int], window: int = 32, min_repeats: int = 4) -> bool:
        """True when fine; flags a tail that repeats one short pattern ``min_repeats`` times."""
        tail = tokens[-window:]
        for period in range(1, max(2, len(tail) // min_repeats)):
            if len(tail) >= period * min_repeats and all(
                    tail[-1 - i] == tail[-1 - i - period] for i in range(period * (min_repeats - 1))):
                self.anomaly(uuid, f"REPETITION period={period}")
                return False
        return True

    def anomaly(self, uuid: str, what: str) -> Optional[str]:
        if not self.enabled:
            return None
        self.record(uuid, SeqEvent.ANOMALY, note=what)
        text = json.dumps({"uuid": uuid, "anomaly": what,
                           "events": [(round(t, 6), SeqEvent(e).name, v, n) for t, e, v, n in self._rings[uuid]]})
        self.dumps.append(text)
        if self.dump_dir:
            os.makedirs(self.dump_dir, exist_ok=True)
            path = os.path.join(self.dump_dir, f"lifespan_{uuid}.json")
            with open(path, "w") as f:
                f.write(text)
            return path
        return None
