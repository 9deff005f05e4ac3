"""Stage a converted checkpoint into fast local storage (tmpfs) before workers map it.

A staged store is a directory of shard files plus ``MANIFEST.json`` with each file's size and BLAKE2 digest
and a digest over the whole listing.  Staging is idempotent and crash safe: files are copied to a temporary
name and renamed, the manifest is written last, and a later start re-uses a complete, matching store
(verifying sizes always and digests on request) or finishes an interrupted one.  ``partition=(i, n)`` stages
only the i-th of n shard groups (a node of a distributed weight store keeps 1/n of the checkpoint).

Reference parity: batchgen/server/weight_store_staging.py (tmpfs staging with manifest hashing).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

MANIFEST = "MANIFEST.json"


def _digest(path: str, chunk: int = 8 << 20) -> str:
    h = hashlib.blake2b(digest_size=16)
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def _listing_digest(files: Dict[str, Dict[str, object]]) -> str:
    h = hashlib.blake2b(digest_size=16)
    for name in sorted(files):
        h.update(f"{name}:{files[name]['bytes']}:{files[name]['digest']};".encode())
    return h.hexdigest()


@dataclass
class StagedStore:
    root: str
    files: Dict[str, Dict[str, object]]
    listing_digest: str
    reused: bool
    copied_bytes: int


def _source_files(src_dir: str, partition: Optional[Tuple[int, int]]) -> List[str]:
    stems = sorted({os.path.splitext(f)[0] for f in os.listdir(src_dir) if f.endswith(".bin")})
    if partition is not None:
        i, n = partition
        if not 0 <= i < n:
            raise ValueError("partition index out of range")
        stems = stems[i::n]
    out = []
    for s in stems:
        for ext in (".bin", ".json"):
            p = os.path.join(src_dir, s + ext)
            if not os.path.exists(p):
                raise FileNotFoundError(f"{p} is missing: every shard needs its .bin and .json")
            out.append(s + ext)
    return out


def verify_store(root: str, check_digests: bool = False) -> Optional[str]:
    """None if the staged store is complete and consistent, else the first problem found."""
    mpath = os.path.join(root, MANIFEST)
    if not os.path.exists(mpath):
        return "no manifest"
    with open(mpath) as f:
        man = json.load(f)
    if man.get("listing_digest") != _listing_digest(man["files"]):
        return "manifest listing digest mismatch"
    for name, meta in man["files"].items():
        p = os.path.join(root, name)
        if not os.path.exists(p):
            return f"{name} is missing"
        if os.path.getsize(p) != meta["bytes"]:
            return f"{name} has {os.path.getsize(p)} bytes, manifest says {meta['bytes']}"
        if check_digests and _digest(p) != meta["digest"]:
            return f"{name} digest mismatch"
    return None


def stage_store(src_dir: str, dst_root: str, partition: Optional[Tuple[int, int]] = None,
                check_digests: bool = False) -> StagedStore:
    names = _source_files(src_dir, partition)
    os.makedirs(dst_root, exist_ok=True)
    want = {n: {"bytes": os.path.getsize(os.path.join(src_dir, n)), "digest": _digest(os.path.join(src_dir, n))}
            for n in names}
    listing = _listing_digest(want)
    mpath = os.path.join(dst_root, MANIFEST)
    if os.path.exists(mpath):
        with open(mpath) as f:
            have = json.load(f)
        if have.get("listing_digest") == listing and verify_store(dst_root, check_digests) is None:
            return StagedStore(dst_root, have["files"], listing, True, 0)
        os.unlink(mpath)                       # stale or damaged: restage below, manifest goes last again
    copied = 0
    for n, meta in want.items():
        dst = os.path.join(dst_root, n)
        if os.path.exists(dst) and os.path.getsize(dst) == meta["bytes"] and (not check_digests or _digest(dst) == meta["digest"]):
            continue
        tmp = dst + f".tmp-{os.getpid()}"
        shutil.copyfile(os.path.join(src_dir, n), tmp)
        os.replace(tmp, dst)
        copied += int(meta["bytes"])
    for stale in os.listdir(dst_root):
        if stale != MANIFEST and stale not in want:
            os.unlink(os.path.join(dst_root, stale))
    tmp = mpath + f".tmp-{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump({"files": want, "listing_digest": listing, "source": os.path.abspath(src_dir),
                   "partition": list(partition) if partition else None}, f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, mpath)
    return StagedStore(dst_root, want, listing, False, copied)
