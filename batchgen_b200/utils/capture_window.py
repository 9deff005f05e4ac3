"""Profiler capture windows and allocator history for a serving worker.

``CaptureWindow`` brackets a range of engine steps with ``cudaProfilerStart`` / ``cudaProfilerStop`` so that an external
profiler attached with "capture range = profiler API" records exactly those steps of a long-running worker
(``BATCHGEN_PROFILE_STEPS=first:last``, step numbers counted from the worker's first step).

``MemoryHistory`` turns on the caching allocator's event history and writes a snapshot file on demand (the worker
writes one when a step dies of an out-of-memory error; ``BATCHGEN_MEMORY_HISTORY=<directory>``).

Reference parity: the worker's profiler capture windows and memory-history dumps (batchgen/profiling helpers used by
batchgen/batchgen_worker.py).
"""
from __future__ import annotations

import os
import time
from typing import Callable, Optional, Tuple


def parse_window(spec: str) -> Optional[Tuple[int, int]]:
    """"first:last" (inclusive, first >= 0, last >= first) -> (first, last); empty / malformed -> None."""
    if not spec:
        return None
    try:
        a, b = spec.split(":")
        first, last = int(a), int(b)
    except ValueError:
        return None
    return (first, last) if 0 <= first <= last else None


class CaptureWindow:
    def __init__(self, window: Optional[Tuple[int, int]], start: Optional[Callable[[], None]] = None,
                 stop: Optional[Callable[[], None]] = None):
        self.window = window
        self.step = 0
        self.active = False
        self.done = False
        if start is None or stop is None:
            import torch
            cuda = torch.cuda.is_available()
            start = start or ((lambda: torch.cuda.profiler.start()) if cuda else (lambda: None))
            stop = stop or ((lambda: (torch.cuda.synchronize(), torch.cuda.profiler.stop())) if cuda else (lambda: None))
        self._start, self._stop = start, stop

    @classmethod
    def from_env(cls) -> "CaptureWindow":
        return cls(parse_window(os.environ.get("BATCHGEN_PROFILE_STEPS", "")))

    def before_step(self) -> None:
        if self.window and not self.done and not self.active and self.step == self.window[0]:
            self._start()
            self.active = True

    def after_step(self) -> None:
        if self.active and self.step == self.window[1]:
            self._stop()
            self.active, self.done = False, True
        self.step += 1


class MemoryHistory:
    def __init__(self, directory: str = "", max_entries: int = 100_000):
        self.directory = directory
        self.enabled = False
        if directory:
            import torch
            if torch.cuda.is_available() and hasattr(torch.cuda.memory, "_record_memory_history"):
                os.makedirs(directory, exist_ok=True)
                torch.cuda.memory._record_memory_history(max_entries=max_entries)
                self.enabled = True

    @classmethod
    def from_env(cls) -> "MemoryHistory":
        return cls(os.environ.get("BATCHGEN_MEMORY_HISTORY", ""))

    def dump(self, tag: str) -> Optional[str]:
        """Write the allocator snapshot; returns the file path (None when the history is off)."""
        if not self.enabled:
            return None
        import torch
        path = os.path.join(self.directory, f"memory_{tag}_{os.getpid()}_{int(time.time())}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        return path
