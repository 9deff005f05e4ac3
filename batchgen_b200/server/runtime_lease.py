"""Run identity and lane leases: how several servers share one machine without colliding.

A *lane* is the set of things one server run owns exclusively: its GPUs (by UUID), its TCP ports and its
writable directories.  The launcher reserves a lane by taking an exclusive ``flock`` on one lock file per
resource under a private lock root (``LaneReservation.reserve``), writes a manifest that names the open
descriptors, and starts the server with those descriptors inherited.  The server adopts the lane
(``LaneLease.adopt``): it recomputes from its own arguments which resources it is about to use, checks that
the manifest covers exactly those, that every descriptor really is the lock file of its resource, takes
the locks again on the inherited descriptions and keeps them, non-inheritable, until it exits.  The kernel
drops the locks when the process dies, so a crashed run never blocks the next one.

``RunIdentity`` names the objects one run creates (shared-memory segments, runtime directory) so that two
runs of the same instance never share them and stale ones can be found by prefix.

Reference parity: batchgen/server/runtime_lease.py:1-246 (lease validation and ownership),
runtime_identity.py:1-79 (names), scripts/lane_runtime.py (launcher side).
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import re
import secrets
import stat
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Set

MANIFEST_VERSION = 1
MAX_MANIFEST_BYTES = 64 * 1024
DEFAULT_LOCK_ROOT = Path(tempfile.gettempdir()) / "batchgen-b200-lanes"


class LaneLeaseError(RuntimeError):
    pass


# ---------------------------------------------------------------------------------------------- identity
@dataclass(frozen=True)
class RunIdentity:
    instance_id: str      # stable name of the deployment ([a-z0-9][a-z0-9_-]{0,47})
    run_id: str           # 32 hex characters, new for every start
    mode: str = "exclusive"   # exclusive: the machine is ours; shared: a lane lease is mandatory

    @classmethod
    def create(cls, instance_id: str, mode: str = "exclusive", run_id: Optional[str] = None) -> "RunIdentity":
        if mode not in ("exclusive", "shared"):
            raise ValueError("mode must be 'exclusive' or 'shared'")
        if not re.fullmatch(r"[a-z0-9][a-z0-9_-]{0,47}", instance_id or ""):
            raise ValueError("instance_id must match [a-z0-9][a-z0-9_-]{0,47}")
        run_id = secrets.token_hex(16) if run_id is None else run_id
        if not re.fullmatch(r"[0-9a-f]{32}", run_id):
            raise ValueError("run_id must be 32 lowercase hexadecimal characters")
        return cls(instance_id, run_id, mode)

    @property
    def prefix(self) -> str:
        return f"bgb200_{self.instance_id}_{self.run_id}"

    def shm_name(self, what: str) -> str:
        """Name of a node-shared segment of this run (host KV, prefix index, token book, ...)."""
        return f"{self.prefix}.{what}"

    @property
    def runtime_dir(self) -> Path:
        return Path(tempfile.gettempdir()) / self.prefix


# ---------------------------------------------------------------------------------------------- resources
def resource_names(gpu_uuids: Sequence[str], ports: Iterable[int], paths: Iterable[os.PathLike]) -> Set[str]:
    out = {f"gpu:{u}" for u in gpu_uuids}
    out |= {f"port:{int(p)}" for p in ports}
    out |= {"path:" + hashlib.sha256(str(Path(p).expanduser().resolve()).encode()).hexdigest() for p in paths}
    return out


def _lock_file(root: Path, resource: str) -> Path:
    return root / (hashlib.sha256(resource.encode()).hexdigest() + ".lock")


def _check_root(root: Path) -> Path:
    if root.is_symlink() or not root.is_dir():
        raise LaneLeaseError(f"lock root {root} is not a directory")
    st = root.stat()
    if st.st_uid != os.geteuid() or st.st_mode & 0o077:
        raise LaneLeaseError(f"lock root {root} must belong to this user with mode 0700")
    return root.resolve()


# ---------------------------------------------------------------------------------------------- launcher side
class LaneReservation:
    """Launcher side: exclusive locks on every resource of a lane plus the manifest that hands them over."""

    def __init__(self, manifest_fd: int, fds: Dict[str, int]):
        self.manifest_fd, self.fds = manifest_fd, fds

    @classmethod
    def reserve(cls, instance_id: str, resources: Iterable[str], lock_root: Path = DEFAULT_LOCK_ROOT) -> "LaneReservation":
        lock_root.mkdir(mode=0o700, parents=True, exist_ok=True)
        root = _check_root(lock_root)
        fds: Dict[str, int] = {}
        try:
            for r in sorted(set(resources)):
                fd = os.open(_lock_file(root, r), os.O_RDWR | os.O_CREAT, 0o600)
                fds[r] = fd
                try:
                    fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                except OSError as e:
                    raise LaneLeaseError(f"{r} is held by another run") from e
                os.set_inheritable(fd, True)
            mfd = os.memfd_create("bgb200-lane-manifest") if hasattr(os, "memfd_create") else \
                os.open(tempfile.mkstemp(prefix="lane-", dir=root)[1], os.O_RDWR)
            body = json.dumps({"version": MANIFEST_VERSION, "instance_id": instance_id, "resources": fds}).encode()
            os.pwrite(mfd, body, 0)
            os.set_inheritable(mfd, True)
            return cls(mfd, fds)
        except BaseException:
            for fd in fds.values():
                os.close(fd)
            raise

    def release(self) -> None:
        for fd in list(self.fds.values()) + [self.manifest_fd]:
            try:
                os.close(fd)
            except OSError:
                pass
        self.fds = {}


# ---------------------------------------------------------------------------------------------- server side
class LaneLease:
    """Server side: the adopted descriptors; the lane is ours until ``release`` or process exit."""

    def __init__(self, manifest_fd: int, fds: List[int]):
        self._manifest_fd, self._fds = manifest_fd, fds

    @property
    def held(self) -> int:
        return len(self._fds)

    @classmethod
    def adopt(cls, manifest_fd: int, instance_id: str, expected: Set[str], lock_root: Path = DEFAULT_LOCK_ROOT) -> "LaneLease":
        try:
            st = os.fstat(manifest_fd)
        except OSError as e:
            raise LaneLeaseError("the manifest descriptor is not open") from e
        if not stat.S_ISREG(st.st_mode) or st.st_uid != os.geteuid() or not 0 < st.st_size <= MAX_MANIFEST_BYTES:
            raise LaneLeaseError("the manifest must be a small regular file of this user")
        try:
            m = json.loads(os.pread(manifest_fd, st.st_size, 0).decode())
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise LaneLeaseError("the manifest is not valid JSON") from e
        if not isinstance(m, dict) or m.get("version") != MANIFEST_VERSION:
            raise LaneLeaseError("unsupported manifest version")
        if m.get("instance_id") != instance_id:
            raise LaneLeaseError("the lease was issued to another instance")
        res = m.get("resources")
        if not isinstance(res, dict) or set(res) != set(expected):
            missing, extra = sorted(set(expected) - set(res or ())), sorted(set(res or ()) - set(expected))
            raise LaneLeaseError(f"the lease does not cover this server's resources (missing {missing}, extra {extra})")
        root = _check_root(lock_root)
        fds: List[int] = []
        for r in sorted(expected):
            fd = res[r]
            if not isinstance(fd, int) or fd < 0 or fd == manifest_fd or fd in fds:
                raise LaneLeaseError(f"bad descriptor for {r}")
            try:
                fst = os.fstat(fd)
                target = Path(os.readlink(f"/proc/self/fd/{fd}")).resolve()
            except OSError as e:
                raise LaneLeaseError(f"the descriptor of {r} is not open") from e
            if not stat.S_ISREG(fst.st_mode) or fst.st_uid != os.geteuid() or target != _lock_file(root, r):
                raise LaneLeaseError(f"the descriptor of {r} is not its lock file")
            fds.append(fd)
        for fd in fds:
            try:
                fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)     # same open description as the launcher's lock
            except OSError as e:
                raise LaneLeaseError("a lane resource is locked by someone else") from e
            os.set_inheritable(fd, False)
        os.set_inheritable(manifest_fd, False)
        return cls(manifest_fd, fds)

    def release(self) -> None:
        for fd in self._fds + [self._manifest_fd]:
            try:
                os.close(fd)
            except OSError:
                pass
        self._fds = []


def expected_for_server(gpu_uuids: Sequence[str], listen_port: int, dist_port: int, storage_path: os.PathLike,
                        extra_paths: Iterable[os.PathLike] = ()) -> Set[str]:
    """The resources a server with these arguments is about to use; ``CUDA_VISIBLE_DEVICES`` must list exactly
    the leased GPUs in the same order."""
    visible = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
    if visible and list(gpu_uuids) != visible:
        raise LaneLeaseError("the leased GPUs must equal CUDA_VISIBLE_DEVICES, in order")
    if any(not u.startswith("GPU-") for u in gpu_uuids):
        raise LaneLeaseError("GPUs are leased by UUID")
    return resource_names(gpu_uuids, [listen_port, dist_port], [storage_path, *extra_paths])
