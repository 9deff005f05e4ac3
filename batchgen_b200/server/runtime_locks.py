"""Runtime locks and run-scoped cleanup of one server instance on a host.

* The *host lock* (``<runtime_root>/host.lock``) serialises start-up and reclamation on a host; the
  *instance lock* (``<runtime_dir>/instance.lock``) is held for the life of a server so that a second server
  cannot start in the same runtime directory.
* Every worker holds a shared *run lock* on ``<runtime_dir>/run.lock``.  Node-shared objects (shared-memory
  segments, sockets) carry the run id in their name; a later start that can take the run lock exclusively
  knows the run is dead and removes what it left behind.

Locks are ``flock`` locks: the kernel drops them when the holder dies, however it dies.

Reference parity: batchgen/server/runtime_locks.py:25-200 (RuntimeLocks, hold_run_lock, list_run_named_objects,
reclaim_dead_runs); batchgen/server/runtime_lease.py (per-resource lane leases).
"""
from __future__ import annotations

import fcntl
import os
from pathlib import Path
from typing import BinaryIO, Iterable, List, Optional


class RuntimeLockError(RuntimeError):
    pass


def _lock(path: Path, exclusive: bool, blocking: bool) -> BinaryIO:
    path.parent.mkdir(parents=True, exist_ok=True)
    f = open(path, "ab+")
    try:
        fcntl.flock(f.fileno(), (fcntl.LOCK_EX if exclusive else fcntl.LOCK_SH) | (0 if blocking else fcntl.LOCK_NB))
    except BlockingIOError:
        f.close()
        raise RuntimeLockError(f"{path} is held by another process") from None
    return f


class RuntimeLocks:
    def __init__(self, host_file: BinaryIO, instance_file: BinaryIO):
        self._host, self._instance = host_file, instance_file

    @classmethod
    def acquire(cls, runtime_root: os.PathLike, runtime_dir: os.PathLike) -> "RuntimeLocks":
        """Take the host lock (wait), then the instance lock (fail if another server owns the directory); the
        host lock is released once the instance lock is held."""
        host = _lock(Path(runtime_root) / "host.lock", exclusive=True, blocking=True)
        try:
            inst = _lock(Path(runtime_dir) / "instance.lock", exclusive=True, blocking=False)
        except RuntimeLockError:
            host.close()
            raise
        fcntl.flock(host.fileno(), fcntl.LOCK_UN)
        return cls(host, inst)

    def close(self) -> None:
        for f in (self._instance, self._host):
            try:
                f.close()
            except OSError:
                pass


def hold_run_lock(runtime_dir: os.PathLike, *, create: bool = False) -> BinaryIO:
    """Shared lock that every process of a run holds for its whole life."""
    path = Path(runtime_dir) / "run.lock"
    if not create and not path.exists():
        raise RuntimeLockError(f"{path} does not exist: the server did not start this run")
    return _lock(path, exclusive=False, blocking=True)


def release_run_lock(f: Optional[BinaryIO]) -> None:
    if f is not None:
        f.close()


def run_is_dead(runtime_dir: os.PathLike) -> bool:
    """True if no process holds the run lock any more (taken exclusively without waiting, then dropped)."""
    path = Path(runtime_dir) / "run.lock"
    if not path.exists():
        return True
    try:
        _lock(path, exclusive=True, blocking=False).close()
        return True
    except RuntimeLockError:
        return False


def list_run_named_objects(run_id: str, roots: Iterable[os.PathLike] = ("/dev/shm",)) -> List[Path]:
    out: List[Path] = []
    for root in roots:
        p = Path(root)
        if p.is_dir():
            out.extend(sorted(q for q in p.iterdir() if run_id in q.name))
    return out


def reclaim_dead_runs(runtime_root: os.PathLike, roots: Iterable[os.PathLike] = ("/dev/shm",)) -> List[str]:
    """Under the host lock: for every run directory whose run lock nobody holds, remove its named objects and
    the directory's lock files.  Returns the reclaimed run ids."""
    root = Path(runtime_root)
    reclaimed: List[str] = []
    if not root.is_dir():
        return reclaimed
    host = _lock(root / "host.lock", exclusive=True, blocking=True)
    try:
        for d in sorted(p for p in root.iterdir() if p.is_dir()):
            if (d / "run.lock").exists() and run_is_dead(d):
                for obj in list_run_named_objects(d.name, roots):
                    try:
                        obj.unlink()
                    except OSError:
                        pass
                for name in ("run.lock", "instance.lock"):
                    try:
                        (d / name).unlink()
                    except OSError:
                        pass
                reclaimed.append(d.name)
    finally:
        host.close()
    return reclaimed
