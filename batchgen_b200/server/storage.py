"""Disk store of uploaded files, batch objects and incrementally written outputs.

Layout under ``--storage-path``:  ``files/<id>`` + ``files/<id>.json`` (FileObject), ``batches/<id>.json``
(BatchObject), ``owner.lock`` (flock held by the live server).  Ownership is exclusive: a second server
on the same directory fails to start.  At start-up, batches that a previous server left ``validating`` /
``in_progress`` are orphans: they are marked ``failed`` with a reason and whatever output they had already
flushed is published, so no client waits forever.  Uploads are de-duplicated by SHA-256.

Reference parity: batchgen/server/storage.py (files/batches/outputs, flock ownership, orphan recovery used
at batchgen/server/http_server.py:192-210; incremental fsync'd output docs/server-flags.md:495-512).
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import threading
import time
from typing import Dict, List, Optional

from .io_struct import BatchError, BatchErrors, BatchObject, FileObject


class StorageOwnershipError(RuntimeError):
    pass


class StorageManager:
    def __init__(self, root: str):
        self.root = os.path.abspath(root)
        self.files_dir = os.path.join(self.root, "files")
        self.batches_dir = os.path.join(self.root, "batches")
        os.makedirs(self.files_dir, exist_ok=True)
        os.makedirs(self.batches_dir, exist_ok=True)
        self._lock = threading.RLock()
        self._owner_fd: Optional[int] = None
        self._out_handles: Dict[str, object] = {}

    # ------------------------------------------------------------------ ownership
    def acquire_ownership(self) -> None:
        fd = os.open(os.path.join(self.root, "owner.lock"), os.O_RDWR | os.O_CREAT, 0o644)
        try:
            fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError:
            os.close(fd)
            raise StorageOwnershipError(f"{self.root} is owned by another live server")
        os.ftruncate(fd, 0)
        os.write(fd, str(os.getpid()).encode())
        self._owner_fd = fd

    def release_ownership(self) -> None:
        if self._owner_fd is not None:
            fcntl.flock(self._owner_fd, fcntl.LOCK_UN)
            os.close(self._owner_fd)
            self._owner_fd = None

    # ------------------------------------------------------------------ files
    def _file_path(self, fid: str) -> str:
        return os.path.join(self.files_dir, fid)

    def save_file(self, data: bytes, filename: str, purpose: str = "batch") -> FileObject:
        sha = hashlib.sha256(data).hexdigest()
        with self._lock:
            for f in self.list_files():
                if f.sha256 == sha and f.purpose == purpose and f.filename == filename:
                    return f
            fo = FileObject(bytes=len(data), filename=filename, purpose=purpose, sha256=sha)
            tmp = self._file_path(fo.id) + ".tmp"
            with open(tmp, "wb") as fh:
                fh.write(data)
                fh.flush()
                os.fsync(fh.fileno())
            os.replace(tmp, self._file_path(fo.id))
            self._write_json(self._file_path(fo.id) + ".json", fo.model_dump())
            return fo

    def get_file(self, fid: str) -> Optional[FileObject]:
        p = self._file_path(fid) + ".json"
        if not os.path.exists(p):
            return None
        with open(p) as fh:
            return FileObject(**json.load(fh))

    def read_file(self, fid: str) -> Optional[bytes]:
        p = self._file_path(fid)
        if not os.path.exists(p):
            return None
        with open(p, "rb") as fh:
            return fh.read()

    def list_files(self) -> List[FileObject]:
        out = []
        for n in sorted(os.listdir(self.files_dir)):
            if n.endswith(".json"):
                with open(os.path.join(self.files_dir, n)) as fh:
                    out.append(FileObject(**json.load(fh)))
        return sorted(out, key=lambda f: f.created_at)

    def delete_file(self, fid: str) -> bool:
        with self._lock:
            found = False
            for p in (self._file_path(fid), self._file_path(fid) + ".json"):
                if os.path.exists(p):
                    os.remove(p)
                    found = True
            return found

    # ------------------------------------------------------------------ batches
    def _batch_path(self, bid: str) -> str:
        return os.path.join(self.batches_dir, bid + ".json")

    def save_batch(self, b: BatchObject) -> None:
        with self._lock:
            self._write_json(self._batch_path(b.id), b.model_dump())

    def get_batch(self, bid: str) -> Optional[BatchObject]:
        p = self._batch_path(bid)
        if not os.path.exists(p):
            return None
        with open(p) as fh:
            return BatchObject(**json.load(fh))

    def list_batches(self) -> List[BatchObject]:
        out = []
        for n in os.listdir(self.batches_dir):
            if n.endswith(".json"):
                with open(os.path.join(self.batches_dir, n)) as fh:
                    out.append(BatchObject(**json.load(fh)))
        return sorted(out, key=lambda b: b.created_at)

    # ------------------------------------------------------------------ incremental outputs
    def output_path(self, bid: str) -> str:
        return os.path.join(self.batches_dir, bid + ".out.jsonl")

    def append_output(self, bid: str, item: dict) -> None:
        """Append one result line and fsync it: a crash keeps every completed request."""
        with self._lock:
            fh = self._out_handles.get(bid)
            if fh is None:
                fh = open(self.output_path(bid), "a")
                self._out_handles[bid] = fh
            fh.write(json.dumps(item) + "\n")
            fh.flush()
            os.fsync(fh.fileno())

    def publish_output(self, bid: str) -> Optional[FileObject]:
        """Turn the incremental output into a downloadable file object."""
        with self._lock:
            fh = self._out_handles.pop(bid, None)
            if fh is not None:
                fh.close()
            p = self.output_path(bid)
            if not os.path.exists(p):
                return None
            with open(p, "rb") as f:
                data = f.read()
            return self.save_file(data, f"{bid}_output.jsonl", purpose="batch_output")

    # ------------------------------------------------------------------ recovery
    def fail_orphaned_batches(self, reason: str = "server restarted while the batch was in flight") -> List[str]:
        failed = []
        for b in self.list_batches():
            if b.status in ("validating", "in_progress", "finalizing", "cancelling"):
                b.status = "failed"
                b.failed_at = int(time.time())
                b.errors = BatchErrors(data=[BatchError(code="server_restart", message=reason)])
                fo = self.publish_output(b.id)
                if fo is not None:
                    b.output_file_id = fo.id
                self.save_batch(b)
                failed.append(b.id)
        return failed

    @staticmethod
    def _write_json(path: str, obj: dict) -> None:
        tmp = path + ".tmp"
        with open(tmp, "w") as fh:
            json.dump(obj, fh)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, path)
