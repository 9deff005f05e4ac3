"""What a server takes before it serves and keeps until it exits: the run identity, the runtime locks, the lane
lease handed over by a launcher, and the reclamation of what dead runs left behind.  Workers join the run by taking
the shared run lock (``join_run``), so that a later start can tell a dead run from a live one.

Reference parity: batchgen/launch_http_server.py:60-111 (identity + locks before the server starts),
batchgen/server/runtime_locks.py, batchgen/server/runtime_lease.py.
"""
from __future__ import annotations

import os
import tempfile
from pathlib import Path
from typing import BinaryIO, List, Optional

from . import runtime_lease, runtime_locks


class RunGuard:
    def __init__(self, identity: runtime_lease.RunIdentity, runtime_root: Path, run_dir: Path,
                 locks: runtime_locks.RuntimeLocks, run_lock: BinaryIO, lease: Optional[runtime_lease.LaneLease],
                 reclaimed: List[str]):
        self.identity, self.runtime_root, self.run_dir = identity, runtime_root, run_dir
        self.locks, self.run_lock, self.lease, self.reclaimed = locks, run_lock, lease, reclaimed

    def close(self) -> None:
        runtime_locks.release_run_lock(self.run_lock)
        self.run_lock = None
        if self.lease is not None:
            self.lease.release()
            self.lease = None
        self.locks.close()


def default_runtime_root() -> Path:
    return Path(tempfile.gettempdir()) / "batchgen-b200-runtime"


def acquire(args) -> RunGuard:
    """Called once by the launcher process.  Order: reclaim dead runs (under the host lock), take the instance lock
    of ``--instance-id`` (a second server of the same instance fails here), create this run's directory and hold its
    run lock, then adopt the lane lease if a launcher passed one (``--lane-manifest-fd``; mandatory in shared
    mode).  Sets ``args.runtime_dir`` and ``args.run_id`` for the workers."""
    instance = args.instance_id or f"port{args.port}"
    identity = runtime_lease.RunIdentity.create(instance, mode=args.run_mode)
    root = Path(args.runtime_root) if args.runtime_root else default_runtime_root()
    root.mkdir(parents=True, exist_ok=True)
    reclaimed = runtime_locks.reclaim_dead_runs(root)
    inst_dir = root / f"instance-{instance}"
    inst_dir.mkdir(exist_ok=True)
    locks = runtime_locks.RuntimeLocks.acquire(root, inst_dir)
    try:
        run_dir = root / identity.prefix
        run_dir.mkdir(exist_ok=True)
        run_lock = runtime_locks.hold_run_lock(run_dir, create=True)
        lease = None
        if args.lane_manifest_fd >= 0:
            gpus = [g for g in (args.lane_gpus or os.environ.get("CUDA_VISIBLE_DEVICES", "")).split(",") if g.strip()]
            dist_port = int(str(args.dist_init_addr).rsplit(":", 1)[-1])
            expected = runtime_lease.expected_for_server(gpus, args.port, dist_port, args.storage_path)
            lock_root = Path(args.lane_lock_root) if args.lane_lock_root else runtime_lease.DEFAULT_LOCK_ROOT
            lease = runtime_lease.LaneLease.adopt(args.lane_manifest_fd, instance, expected, lock_root)
        elif identity.mode == "shared":
            raise runtime_lease.LaneLeaseError("--run-mode shared needs a lane lease (--lane-manifest-fd)")
    except Exception:
        locks.close()
        raise
    args.runtime_dir, args.run_id = str(run_dir), identity.run_id
    return RunGuard(identity, root, run_dir, locks, run_lock, lease, reclaimed)


def join_run(args) -> Optional[BinaryIO]:
    """Worker side: hold the run's shared lock for the life of the process (None when the server runs unguarded,
    e.g. in-process tests)."""
    d = getattr(args, "runtime_dir", "")
    if not d:
        return None
    return runtime_locks.hold_run_lock(d)
