"""Was a worker killed by the kernel's out-of-memory killer?

A worker that dies with SIGKILL and no Python traceback is most often a host-memory kill (pinned KV, weight staging).
The kernel says so in its log; this module finds the line that names one of our process ids, so that the server's
failure message reads "killed by the kernel OOM killer" instead of "exited with code -9".

Reference parity: batchgen/server/worker_manager.py:2072-2250 (host OOM attribution from the kernel log).
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Iterable, List, Optional

_PATTERNS = (
    re.compile(r"Out of memory: Killed process (?P<pid>\d+) \((?P<comm>[^)]*)\)(?P<rest>.*)"),
    re.compile(r"oom-kill:.*?task=(?P<comm>[^,]*),pid=(?P<pid>\d+)(?P<rest>.*)"),
    re.compile(r"Memory cgroup out of memory: Killed process (?P<pid>\d+) \((?P<comm>[^)]*)\)(?P<rest>.*)"),
)
_RSS = re.compile(r"anon-rss:(\d+)kB")


@dataclass
class OomRecord:
    pid: int
    comm: str
    anon_rss_kb: Optional[int]
    line: str

    def describe(self) -> str:
        rss = f", {self.anon_rss_kb / 1048576:.1f} GiB anonymous memory" if self.anon_rss_kb else ""
        return f"process {self.pid} ({self.comm}) was killed by the kernel OOM killer{rss}"


def scan(lines: Iterable[str], pids: Iterable[int]) -> Optional[OomRecord]:
    """The last kernel-log line that reports an OOM kill of one of ``pids``."""
    want = set(int(p) for p in pids)
    found = None
    for line in lines:
        for pat in _PATTERNS:
            m = pat.search(line)
            if m and int(m.group("pid")) in want:
                rss = _RSS.search(m.group("rest") or "")
                found = OomRecord(int(m.group("pid")), m.group("comm"), int(rss.group(1)) if rss else None, line.strip())
    return found


def read_kernel_log(path: str = "/dev/kmsg", max_bytes: int = 1 << 20) -> List[str]:
    """Recent kernel messages without blocking; an unreadable log (no privilege) gives an empty list."""
    out: List[str] = []
    try:
        fd = os.open(path, os.O_RDONLY | os.O_NONBLOCK)
    except OSError:
        return out
    try:
        got = 0
        while got < max_bytes:
            try:
                rec = os.read(fd, 8192)
            except BlockingIOError:
                break
            except OSError:
                break
            if not rec:
                break
            got += len(rec)
            out.append(rec.decode("utf-8", "replace"))
    finally:
        os.close(fd)
    if out and path != "/dev/kmsg":                       # a plain file: records are lines
        out = "".join(out).splitlines()
    return out


def attribute(pids: Iterable[int], log_path: str = "/dev/kmsg") -> Optional[OomRecord]:
    return scan(read_kernel_log(log_path), pids)
