"""Where a CUDA tensor meets an operator whose hand-written sm_100a kernel does not cover its geometry.

The production geometries (DeepSeek / GLM / Kimi / GPT-OSS shapes) all have kernels.  Test-sized models
(tiny latent widths, odd head counts) do not; for them a library implementation (cuBLAS ``bmm`` / ``mm``
and eager softmax) exists as a numerics cross-check.  It must never be reached silently on a GPU: by default
``library_fallback`` raises ``KernelError`` and names the operator and the geometry.  Tests that run tiny
geometries on a GPU opt in explicitly with ``allow_library_fallback()`` (or ``BG_ALLOW_LIBRARY_FALLBACK=1``).
"""
from __future__ import annotations

import contextlib
import os
from collections import Counter

from ._ext import KernelError

_ALLOW = [os.environ.get("BG_ALLOW_LIBRARY_FALLBACK", "0") == "1"]
FALLBACKS: Counter = Counter()        # operator -> times the library path ran (while allowed)


def library_fallback(op: str, why: str) -> None:
    """Called right before a library path runs on CUDA tensors."""
    if not _ALLOW[0]:
        raise KernelError(f"{op}: no sm_100a kernel for this geometry ({why}); the library path is off by default "
                          f"on CUDA (enable it for test-sized models with ops.policy.allow_library_fallback())")
    FALLBACKS[op] += 1


@contextlib.contextmanager
def allow_library_fallback(allow: bool = True):
    prev = _ALLOW[0]
    _ALLOW[0] = allow
    try:
        yield
    finally:
        _ALLOW[0] = prev


def set_library_fallback(allow: bool) -> None:
    _ALLOW[0] = bool(allow)
