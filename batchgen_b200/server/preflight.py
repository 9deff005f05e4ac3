"""Fail-closed preflights run before the server binds its port.

* launch readiness — storage and checkpoint paths reachable and writable, the HTTP port free;
* runtime preflight — the dependency contract of the chosen model: the in-tree kernel library exists (and was
  built for sm_100a) whenever a GPU will be used, the GPU is a compute-capability 10.x part, torch has the
  collectives backend the world size needs;
* host-memory preflight — offloaded experts + host KV fit ``MemTotal``.

Reference parity: batchgen/launch_readiness.py, batchgen/runtime_preflight.py:160-337,
batchgen/host_memory_preflight.py.
"""
from __future__ import annotations

import os
import socket
from typing import List


class PreflightError(RuntimeError):
    pass


def mem_total_bytes() -> int:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def launch_readiness(args) -> List[str]:
    out = []
    os.makedirs(args.storage_path, exist_ok=True)
    probe = os.path.join(args.storage_path, ".write_probe")
    try:
        with open(probe, "w") as f:
            f.write("ok")
        os.remove(probe)
    except OSError as e:
        raise PreflightError(f"--storage-path {args.storage_path} is not writable: {e}")
    out.append(f"storage path {args.storage_path} writable")
    if args.converted_ckpt_dir:
        if not any(n.endswith(".bin") for n in os.listdir(args.converted_ckpt_dir)):
            raise PreflightError(f"--converted-ckpt-dir {args.converted_ckpt_dir} holds no converted .bin shards")
        out.append("converted checkpoint present")
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((args.host, args.port))
        except OSError as e:
            raise PreflightError(f"cannot bind {args.host}:{args.port}: {e}")
    out.append(f"port {args.port} free")
    return out


def runtime_preflight(args) -> List[str]:
    import torch
    out = []
    want_gpu = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    if want_gpu:
        from ..ops import _ext
        if not _ext.available():
            raise PreflightError("the sm_100a kernel library is missing: run `python -m batchgen_b200.build`")
        if torch.cuda.device_count() < args.world_size:
            raise PreflightError(f"--world-size {args.world_size} but only {torch.cuda.device_count()} GPU(s) visible")
        major, minor = torch.cuda.get_device_capability(0)
        if major != 10:
            raise PreflightError(f"the kernels are built for sm_100a only; device 0 is sm_{major}{minor}")
        out.append(f"kernel library present, {torch.cuda.device_count()} x sm_{major}{minor}")
        if args.world_size > 1 and not torch.distributed.is_nccl_available():
            raise PreflightError("torch was built without NCCL")
    else:
        if args.world_size > 1 and not torch.distributed.is_gloo_available():
            raise PreflightError("torch was built without gloo")
        out.append("CPU execution (fp32 reference path)")
    return out


def host_memory(args) -> List[str]:
    from ..config import get_model_config
    from ..runtime.planner import host_memory_preflight
    total = mem_total_bytes()
    if total == 0:
        return ["MemTotal unknown: host-memory check skipped"]
    why = host_memory_preflight(get_model_config(args.model), args.engine_config(), total, args.world_size)
    if why:
        raise PreflightError(why)
    return [f"host plan fits MemTotal {total >> 30} GiB"]


def run_all_preflights(args) -> List[str]:
    return launch_readiness(args) + runtime_preflight(args) + host_memory(args)
