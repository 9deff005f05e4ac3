"""In-step kernel trace: which kernel started when, inside a captured decode step.

Every kernel of the decode path stamps (global timer, id) on entry when a trace buffer is installed
(``ops/csrc/common.cuh::pdl_prologue``).  CUDA events cannot be placed between the nodes of a replayed graph, and a
profiler serialises and slows what it measures; the stamps cost one atomic per kernel and show each kernel's *period*
in place: its duration plus the gap until the next stamped kernel starts (time spent in kernels that do not stamp,
e.g. library copies, is charged to the stamped kernel before them).
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Dict, List, Tuple

import torch

FILES = {1: "ops/csrc/elementwise.cu", 2: "ops/csrc/moe_route.cu", 3: "ops/csrc/gemm_fp8_n256.cu",
         4: "ops/csrc/gemm_fp8_swapab.cu", 5: "ops/csrc/gemm_tcgen05.cu", 6: "ops/csrc/head_gemm.cu",
         7: "ops/csrc/mla_decode_persist.cu", 8: "ops/csrc/mla_tcgen05.cuh", 9: "ops/csrc/sampling.cu",
         10: "parallel/csrc/fused_comm.cu", 0: "ops/csrc/mla_tcgen05.cuh"}
SETTERS = ["elementwise", "moe_route", "gemm_fp8_n256", "gemm_fp8_swapab", "gemm_tcgen05", "head_gemm",
           "mla_decode_persist", "mla_tcgen05", "sampling", "fused_comm"]
_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _set_all(ptr: int) -> None:
    from ..ops import _ext
    L = _ext.lib()
    for name in SETTERS:
        fn = getattr(L, f"bg_trace_set_{name}")
        fn.argtypes = [ctypes.c_void_p]
        if fn(ctypes.c_void_p(ptr)) != 0:
            raise RuntimeError(f"bg_trace_set_{name} failed")


def enable(device, capacity: int = 1 << 16) -> torch.Tensor:
    """Install a fresh trace buffer on ``device`` (call on the device's current context).  Returns the buffer."""
    buf = torch.zeros(1 + 2 * capacity, dtype=torch.int64, device=device)     # [n | cap] then (time, id) pairs
    buf.view(torch.int32)[1] = capacity
    torch.cuda.synchronize(device)
    _set_all(buf.data_ptr())
    return buf


def disable(device) -> None:
    torch.cuda.synchronize(device)
    _set_all(0)


def read(buf: torch.Tensor) -> List[Tuple[int, int, int]]:
    """(time in ns, file tag, line) of every recorded kernel entry, in time order."""
    host = buf.cpu()
    n = min(int(host.view(torch.int32)[0]), int(host.view(torch.int32)[1]))
    rec = host[1:1 + 2 * n].view(n, 2).tolist()
    out = [(t, (i >> 16) & 0xFFFF, i & 0xFFFF) for t, i in rec]
    out.sort()
    return out


_names: Dict[Tuple[int, int], str] = {}


def kernel_name(tag: int, line: int) -> str:
    """Name of the ``__global__`` function whose body contains ``line`` of the tagged file."""
    key = (tag, line)
    if key not in _names:
        name = f"{FILES.get(tag, tag)}:{line}"
        try:
            src = open(os.path.join(_PKG, FILES[tag])).read().splitlines()
            for i in range(min(line, len(src)) - 1, -1, -1):
                if "__global__" in src[i]:
                    m = re.search(r"([A-Za-z_]\w*)\s*\(", " ".join(src[i:i + 3]).split("__global__", 1)[1]
                                  .replace("__launch_bounds__", " "))
                    # skip the launch-bounds argument list if the first match is inside it
                    text = " ".join(src[i:i + 4]).split("__global__", 1)[1]
                    text = re.sub(r"__launch_bounds__\s*\([^)]*\)", " ", text)
                    m = re.search(r"([A-Za-z_]\w*)\s*\(", text.replace("void", " ", 1))
                    if m:
                        name = m.group(1)
                    break
        except (OSError, KeyError):
            pass
        _names[key] = name
    return _names[key]


def summarize(records: List[Tuple[int, int, int]]) -> List[Dict[str, object]]:
    """Per kernel: launches and the sum of periods (start to next start), sorted by time share."""
    agg: Dict[str, List[float]] = {}
    for (t0, tag, line), (t1, _, _) in zip(records, records[1:]):
        a = agg.setdefault(kernel_name(tag, line), [0, 0.0])
        a[0] += 1
        a[1] += (t1 - t0) / 1e3
    total = sum(a[1] for a in agg.values()) or 1.0
    rows = [{"kernel": k, "launches": int(a[0]), "us": a[1], "share": a[1] / total} for k, a in agg.items()]
    rows.sort(key=lambda r: -r["us"])
    return rows
