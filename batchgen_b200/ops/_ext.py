"""Loader for the in-tree CUDA kernel library (plain C ABI through ``ctypes``).

The library is ``batchgen_b200/_C/libbg_kernels.so`` (built by ``batchgen_b200.build``).  On a
machine with a GPU a missing library is an error, never a silent fallback: ``lib()`` raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_C" / "libbg_kernels.so"
_STATUS = {}
_SMS = {}


class KernelError(RuntimeError):
    pass


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python -m batchgen_b200.build` (CUDA tensors need the "
                "sm_100a kernel library; there is no eager fallback on the GPU)")
        _LIB = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else 0)
    return _LIB


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def num_sms(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SMS[idx]


def status_word(device=None) -> torch.Tensor:
    """One int32 per device that kernels raise (atomicMax) when a bounded wait expires."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _STATUS[idx]


def check_status(device=None) -> int:
    """Synchronising read of the status word; raises if any kernel reported a timeout."""
    s = int(status_word(device).item())
    if s != 0:
        status_word(device).zero_()
        raise KernelError(f"kernel reported status {s} (bounded wait expired or bad argument)")
    return s


LAUNCHES = {"count": 0}   # kernels of this library launched by this process (bench.py reports it)


def check(rc: int, what: str, kernels: int = 1) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed to launch (code {rc})")
    LAUNCHES["count"] += kernels
