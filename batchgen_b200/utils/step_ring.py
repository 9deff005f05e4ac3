"""A fixed-size ring of the most recent forward events (prefill forwards, decode steps) of an engine.

Writing costs one tuple store; nothing is formatted until somebody asks.  The worker puts the ring's tail into its
fatal message and its heartbeat, so that "what was the engine doing when it died / stalled" has an answer that does
not depend on log level.  Reference parity: batchgen/worker/step_timing.py (forward-event ring),
batchgen/worker/step_observability_engine.py.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Tuple


class StepRing:
    def __init__(self, capacity: int = 256):
        self.capacity = capacity
        self._buf: List[Optional[Tuple[float, str, int, int, float]]] = [None] * capacity
        self._n = 0
        self._last = time.perf_counter()

    def record(self, kind: str, rows: int, tokens: int, seconds: Optional[float] = None) -> None:
        """``seconds``: host time the event took; default: the time since the previous record."""
        now = time.perf_counter()
        if seconds is None:
            seconds = now - self._last
        self._last = now
        self._buf[self._n % self.capacity] = (time.time(), kind, rows, tokens, seconds)
        self._n += 1

    def __len__(self) -> int:
        return min(self._n, self.capacity)

    def tail(self, n: int = 16) -> List[Dict[str, object]]:
        k = min(n, len(self))
        out = []
        for i in range(self._n - k, self._n):
            ts, kind, rows, tokens, sec = self._buf[i % self.capacity]
            out.append({"ts": round(ts, 3), "kind": kind, "rows": rows, "tokens": tokens, "ms": round(sec * 1e3, 3)})
        return out

    def summary(self) -> Dict[str, Dict[str, float]]:
        """Per kind over the ring: events, tokens, mean and worst milliseconds."""
        agg: Dict[str, List[float]] = {}
        for i in range(max(0, self._n - self.capacity), self._n):
            _, kind, _, tokens, sec = self._buf[i % self.capacity]
            a = agg.setdefault(kind, [0, 0, 0.0, 0.0])
            a[0] += 1
            a[1] += tokens
            a[2] += sec
            a[3] = max(a[3], sec)
        return {k: {"events": a[0], "tokens": a[1], "mean_ms": a[2] / a[0] * 1e3, "max_ms": a[3] * 1e3}
                for k, a in agg.items()}
