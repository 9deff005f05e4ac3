"""In-tree build of the native libraries.

Two shared objects are produced next to the sources they come from:

* ``batchgen_b200/_C/libbg_kernels.so`` — every ``.cu`` under ``ops/csrc`` and ``parallel/csrc``
  compiled by ``nvcc`` for ``sm_100a`` only (plain C ABI, loaded with ``ctypes``; no dependency on
  the torch C++ ABI, so a rebuild takes seconds).
* ``batchgen_b200/_C/libbg_core.so`` — the host-side native engine under ``core/csrc`` (weight
  slot ring, host paged KV, prefix-cache coordinator, copy engines), compiled by ``g++``/``nvcc``.

The reference builds its kernels as AOT torch extensions (batchgen_kernels/setup.py:140-586) and
its engine through a DeepSpeed-style op builder (op_builder/core_engine.py:40-158); here one
function does both and caches on a content hash so repeated calls are free.

Usage: ``python -m batchgen_b200.build [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

PKG = Path(__file__).resolve().parent
OUT = PKG / "_C"
KERNEL_DIRS = [PKG / "ops" / "csrc", PKG / "parallel" / "csrc"]
CORE_DIR = PKG / "core" / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-mavx2", "-mfma"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _hash(paths: List[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: List[str], verbose: bool, log: Path) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "a") as f:
        f.write("$ " + " ".join(cmd) + "\n" + r.stdout + "\n")
    if verbose:
        print(r.stdout)
    if r.returncode != 0:
        raise RuntimeError(f"build command failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout[-4000:]}")


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    srcs = [p for d in KERNEL_DIRS if d.exists() for p in sorted(d.glob("*.cu"))]
    hdrs = [p for d in KERNEL_DIRS if d.exists() for p in sorted(list(d.glob("*.cuh")) + list(d.glob("*.h")))]
    so = OUT / "libbg_kernels.so"
    stamp = OUT / "libbg_kernels.hash"
    digest = _hash(srcs + hdrs, " ".join(NVCC_FLAGS))
    if so.exists() and stamp.exists() and stamp.read_text() == digest and not force:
        return so
    log = OUT / "build_kernels.log"
    log.write_text("")
    nvcc = _nvcc()
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_digest = _hash(hdrs, " ".join(NVCC_FLAGS))

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        ostamp = objdir / (src.stem + ".hash")
        d = _hash([src], hdr_digest)
        if obj.exists() and ostamp.exists() and ostamp.read_text() == d and not force:
            return obj
        inc = [f"-I{x}" for x in KERNEL_DIRS if x.exists()]
        _run([nvcc, *NVCC_FLAGS, *inc, "-c", str(src), "-o", str(obj)], verbose, log)
        ostamp.write_text(d)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([nvcc, "-shared", "-o", str(so), *[str(o) for o in objs], "-lcudart"], verbose, log)
    stamp.write_text(digest)
    return so


def build_core(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    if not CORE_DIR.exists():
        return OUT / "libbg_core.so"
    cpp = sorted(CORE_DIR.glob("*.cpp"))
    cu = sorted(CORE_DIR.glob("*.cu"))
    hdrs = sorted(list(CORE_DIR.glob("*.h")) + list(CORE_DIR.glob("*.hpp")))
    so = OUT / "libbg_core.so"
    stamp = OUT / "libbg_core.hash"
    digest = _hash(cpp + cu + hdrs, " ".join(CXX_FLAGS))
    if so.exists() and stamp.exists() and stamp.read_text() == digest and not force:
        return so
    log = OUT / "build_core.log"
    log.write_text("")
    nvcc = _nvcc()
    objdir = OUT / "obj_core"
    objdir.mkdir(exist_ok=True)
    objs = []
    cuda_inc = str(Path(nvcc).resolve().parent.parent / "include")
    for src in cpp:
        obj = objdir / (src.stem + ".o")
        _run(["g++", *CXX_FLAGS, f"-I{CORE_DIR}", f"-I{cuda_inc}", "-c", str(src), "-o", str(obj)], verbose, log)
        objs.append(obj)
    for src in cu:
        obj = objdir / (src.stem + "_cu.o")
        _run([nvcc, *NVCC_FLAGS, f"-I{CORE_DIR}", "-c", str(src), "-o", str(obj)], verbose, log)
        objs.append(obj)
    _run([nvcc, "-shared", "-o", str(so), *[str(o) for o in objs], "-lcudart", "-lpthread"], verbose, log)
    stamp.write_text(digest)
    return so


def build_all(force: bool = False, verbose: bool = False) -> List[Path]:
    return [build_kernels(force, verbose), build_core(force, verbose)]


if __name__ == "__main__":
    paths = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for p in paths:
        print(p, "ok" if p.exists() else "missing")
