"""Node-level launch gates, evaluated before any worker is spawned: every gate either passes or names what is
missing, and waiting gates have deadlines.  ``python -m batchgen_b200.server.launch_readiness --model-dir D
--port P`` runs them stand-alone.

Gates: model directory readable with a converted checkpoint in it, runtime directory writable, listen ports
free, enough free space under the storage root, shared memory (/dev/shm) large enough for the node-shared
regions, GPUs visible (count), and optional paths that must appear within a deadline (network mounts).

Reference parity: batchgen/launch_readiness.py (node gates with deadlines; CLI), batchgen/launch_http_server.py:35-111.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import socket
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence


@dataclass
class GateResult:
    name: str
    ok: bool
    detail: str = ""


@dataclass
class ReadinessReport:
    results: List[GateResult] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return all(r.ok for r in self.results)

    def failures(self) -> List[GateResult]:
        return [r for r in self.results if not r.ok]

    def to_json(self) -> str:
        return json.dumps({"ok": self.ok, "gates": [r.__dict__ for r in self.results]})


def gate_model_dir(path: str) -> GateResult:
    if not os.path.isdir(path):
        return GateResult("model_dir", False, f"{path} is not a directory")
    if not glob.glob(os.path.join(path, "*.json")) or not glob.glob(os.path.join(path, "*.bin")):
        return GateResult("model_dir", False, f"{path} holds no converted checkpoint (*.bin + *.json)")
    if not os.access(path, os.R_OK):
        return GateResult("model_dir", False, f"{path} is not readable")
    return GateResult("model_dir", True, path)


def gate_writable_dir(name: str, path: str) -> GateResult:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.unlink(probe)
        return GateResult(name, True, path)
    except OSError as e:
        return GateResult(name, False, f"{path}: {e}")


def gate_port_free(host: str, port: int) -> GateResult:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return GateResult(f"port_{port}", True)
        except OSError as e:
            return GateResult(f"port_{port}", False, f"{host}:{port} is taken ({e.strerror})")


def gate_free_space(name: str, path: str, need_bytes: int) -> GateResult:
    try:
        free = shutil.disk_usage(path).free
    except OSError as e:
        return GateResult(name, False, f"{path}: {e}")
    return GateResult(name, free >= need_bytes, f"{free} bytes free under {path}, {need_bytes} needed")


def gate_gpu_count(want: int, count_fn: Optional[Callable[[], int]] = None) -> GateResult:
    if count_fn is None:
        def count_fn():
            import torch
            return torch.cuda.device_count()
    have = count_fn()
    return GateResult("gpus", have >= want, f"{have} visible, {want} needed")


def gate_path_appears(path: str, deadline_s: float, poll_s: float = 0.2,
                      clock: Callable[[], float] = time.monotonic, sleep: Callable[[float], None] = time.sleep) -> GateResult:
    end = clock() + deadline_s
    while True:
        if os.path.exists(path):
            return GateResult(f"path:{path}", True)
        if clock() >= end:
            return GateResult(f"path:{path}", False, f"did not appear within {deadline_s} s")
        sleep(poll_s)


def check_node(model_dir: Optional[str], runtime_dir: str, storage_dir: str, host: str, ports: Sequence[int],
               shm_bytes: int = 0, storage_bytes: int = 0, gpus: int = 0, wait_paths: Sequence[str] = (),
               wait_deadline_s: float = 60.0, gpu_count_fn=None) -> ReadinessReport:
    rep = ReadinessReport()
    for p in wait_paths:
        rep.results.append(gate_path_appears(p, wait_deadline_s))
    if model_dir:
        rep.results.append(gate_model_dir(model_dir))
    rep.results.append(gate_writable_dir("runtime_dir", runtime_dir))
    rep.results.append(gate_writable_dir("storage_dir", storage_dir))
    for port in ports:
        rep.results.append(gate_port_free(host, port))
    if shm_bytes:
        rep.results.append(gate_free_space("shm", "/dev/shm", shm_bytes))
    if storage_bytes:
        rep.results.append(gate_free_space("storage_space", storage_dir, storage_bytes))
    if gpus:
        rep.results.append(gate_gpu_count(gpus, gpu_count_fn))
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="node launch gates")
    ap.add_argument("--model-dir")
    ap.add_argument("--runtime-dir", default="/tmp/batchgen_b200/run")
    ap.add_argument("--storage-dir", default="/tmp/batchgen_b200/storage")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, action="append", default=[])
    ap.add_argument("--gpus", type=int, default=0)
    ap.add_argument("--shm-bytes", type=int, default=0)
    a = ap.parse_args(argv)
    rep = check_node(a.model_dir, a.runtime_dir, a.storage_dir, a.host, a.port, shm_bytes=a.shm_bytes, gpus=a.gpus)
    print(rep.to_json())
    return 0 if rep.ok else 1


if __name__ == "__main__":
    sys.exit(main())
