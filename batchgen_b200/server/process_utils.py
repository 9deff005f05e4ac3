"""Process plumbing for server and workers: die with the parent, signal handling, huge-page sizing.

* ``die_with_parent``: ``prctl(PR_SET_PDEATHSIG, SIGKILL)`` so that a worker never outlives the server that
  spawned it (a worker blocked in a collective would otherwise keep its GPU memory forever); re-checks the
  parent after arming, because the parent may have died in between.
* ``install_termination_handlers``: SIGTERM/SIGINT run the callback once, SIGQUIT dumps all thread stacks.
* ``hugepage_plan``: how a host region of a given size should be backed (1 GiB / 2 MiB / base pages).

Reference parity: batchgen/server/process_utils.py:38 (die_with_parent), :323-350 (huge-page sizing table).
"""
from __future__ import annotations

import ctypes
import faulthandler
import os
import signal
import sys
import threading
from dataclasses import dataclass
from typing import Callable, Optional

PR_SET_PDEATHSIG = 1


def die_with_parent(sig: int = signal.SIGKILL, expected_parent: Optional[int] = None) -> bool:
    """Arm the parent-death signal.  Returns False where prctl is unavailable.  If the parent is already gone
    (re-parented to init or another pid than ``expected_parent``) the process exits at once."""
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        if libc.prctl(PR_SET_PDEATHSIG, int(sig), 0, 0, 0) != 0:
            return False
    except OSError:
        return False
    ppid = os.getppid()
    if ppid == 1 or (expected_parent is not None and ppid != expected_parent):
        os._exit(1)
    return True


def install_termination_handlers(on_terminate: Callable[[int], None], dump_stacks_on_quit: bool = True) -> None:
    fired = threading.Event()

    def handler(signum, _frame):
        if not fired.is_set():
            fired.set()
            on_terminate(signum)

    for s in (signal.SIGTERM, signal.SIGINT):
        signal.signal(s, handler)
    if dump_stacks_on_quit and hasattr(signal, "SIGQUIT"):
        faulthandler.register(signal.SIGQUIT, file=sys.stderr, all_threads=True, chain=False)


@dataclass(frozen=True)
class HugepagePlan:
    page_bytes: int
    pages: int
    kind: str          # "1g" | "2m" | "base"

    @property
    def bytes(self) -> int:
        return self.page_bytes * self.pages


def hugepage_plan(region_bytes: int, free_1g: int = 0, free_2m: int = 0) -> HugepagePlan:
    """Largest page size whose free pool covers the whole region (partial huge backing is never used: a
    region that straddles page sizes cannot be registered for DMA in one piece)."""
    G, M, B = 1 << 30, 2 << 20, 4096
    if free_1g * G >= region_bytes and region_bytes >= G:
        return HugepagePlan(G, -(-region_bytes // G), "1g")
    if free_2m * M >= region_bytes and region_bytes >= M:
        return HugepagePlan(M, -(-region_bytes // M), "2m")
    return HugepagePlan(B, -(-region_bytes // B), "base")


def read_hugepage_pools(meminfo_path: str = "/proc/meminfo", sys_root: str = "/sys/kernel/mm/hugepages") -> dict:
    out = {"free_2m": 0, "free_1g": 0}
    for name, key in (("hugepages-2048kB", "free_2m"), ("hugepages-1048576kB", "free_1g")):
        try:
            with open(os.path.join(sys_root, name, "free_hugepages")) as f:
                out[key] = int(f.read().strip())
        except OSError:
            pass
    return out
