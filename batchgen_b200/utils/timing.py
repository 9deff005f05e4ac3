"""Per-operator CUDA-event timers.

``TimingStats.timed(op, layer)`` brackets a region with an event pair on the current stream; nothing
blocks until ``harvest()`` (called between steps) turns completed pairs into milliseconds.  Summaries
are per op and per (op, layer); ``to_csv`` writes them out.  On CPU tensors wall-clock is used.

Reference parity: batchgen/timing.py:84-454 (``TimingStats``: ``timed(op, layer)`` context managers,
non-blocking ``step_done`` harvest, CSV + per-op/per-layer summaries).
"""
from __future__ import annotations

import contextlib
import csv
import time
from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import torch


class TimingStats:
    def __init__(self, enabled: bool = True, cuda: Optional[bool] = None):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available() if cuda is None else cuda
        self._pending: List[Tuple[str, int, object, object]] = []
        self.totals: Dict[str, float] = defaultdict(float)
        self.counts: Dict[str, int] = defaultdict(int)
        self.by_layer: Dict[Tuple[str, int], float] = defaultdict(float)
        self.steps = 0

    @contextlib.contextmanager
    def timed(self, op: str, layer: int = -1):
        if not self.enabled:
            yield
            return
        if self.cuda:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                self._pending.append((op, layer, e0, e1))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                ms = (time.perf_counter() - t0) * 1e3
                self._add(op, layer, ms)

    def _add(self, op: str, layer: int, ms: float) -> None:
        self.totals[op] += ms
        self.counts[op] += 1
        if layer >= 0:
            self.by_layer[(op, layer)] += ms

    def harvest(self, block: bool = False) -> None:
        """Fold finished event pairs into the totals.  With ``block`` every pending pair is waited for."""
        keep = []
        for op, layer, e0, e1 in self._pending:
            if block:
                e1.synchronize()
            if e1.query():
                self._add(op, layer, e0.elapsed_time(e1))
            else:
                keep.append((op, layer, e0, e1))
        self._pending = keep

    def step_done(self) -> None:
        self.steps += 1
        self.harvest(block=False)

    def summary(self) -> Dict[str, Dict[str, float]]:
        self.harvest(block=True)
        tot = sum(self.totals.values()) or 1.0
        return {op: {"ms": ms, "calls": self.counts[op], "share": ms / tot,
                     "ms_per_step": ms / max(1, self.steps)}
                for op, ms in sorted(self.totals.items(), key=lambda kv: -kv[1])}

    def to_csv(self, path: str) -> None:
        s = self.summary()
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["op", "ms", "calls", "share", "ms_per_step"])
            for op, d in s.items():
                w.writerow([op, f"{d['ms']:.4f}", d["calls"], f"{d['share']:.4f}", f"{d['ms_per_step']:.4f}"])

    def reset(self) -> None:
        self._pending.clear()
        self.totals.clear()
        self.counts.clear()
        self.by_layer.clear()
        self.steps = 0


_NULL = TimingStats(enabled=False)


def null_timer() -> TimingStats:
    return _NULL
