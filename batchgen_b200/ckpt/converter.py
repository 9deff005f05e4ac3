"""Checkpoint converter and reader for the engine's shard format.

A converted shard is two files:

* ``<shard>.bin``  — the tensors of the source shard back to back, raw little-endian bytes, in the
  source's iteration order, no padding;
* ``<shard>.json`` — ``{"file_name": "<shard>.bin", "state_dict": {name: {"dtype", "shape", "offset",
  "byte_size"}}, "total_byte_size": N}``.

This is the format the reference's loader consumes (batchgen/ckpt_converter/ckpt_converter.py:191-262;
dtype names :62-87), so converted checkpoints are interchangeable.  ``ConvertedCheckpoint`` memory-maps
the ``.bin`` files and serves tensors by name without copying; ``loader()`` adapts it to
``models.weights.WeightSource``.  HF DeepSeek-V3 style FP8 checkpoints (``weight`` + ``weight_scale_inv``)
are dequantised on load.

CLI: ``python -m batchgen_b200.ckpt.converter <src_dir> <dst_dir> [--workers N] [--validate]``.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import json
import mmap
import os
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
    torch.float8_e4m3fn: "float8_e4m3fn", torch.int64: "int64", torch.int32: "int32", torch.int8: "int8",
    torch.uint8: "uint8",
}
if hasattr(torch, "float8_e8m0fnu"):
    _DTYPES[torch.float8_e8m0fnu] = "float8_e8m0fnu"
if hasattr(torch, "float4_e2m1fn_x2"):
    _DTYPES[torch.float4_e2m1fn_x2] = "float4_e2m1fn_x2"
_FROM_STR = {v: k for k, v in _DTYPES.items()}


def _load_source(path: str) -> Dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    if path.endswith(".pt"):
        return torch.load(path, weights_only=True, map_location="cpu")
    raise ValueError(f"{path}: only .safetensors and .pt shards can be converted")


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.contiguous()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def convert_shard(src: str, out_dir: str, tensors: Optional[Dict[str, torch.Tensor]] = None) -> str:
    """Convert one shard; returns the path of the metadata file."""
    if tensors is None:
        if not os.path.exists(src):
            raise FileNotFoundError(src)
        tensors = _load_source(src)
    os.makedirs(out_dir, exist_ok=True)
    stem = os.path.basename(src)
    for ext in (".safetensors", ".pt"):
        if stem.endswith(ext):
            stem = stem[: -len(ext)]
    bin_path, meta_path = os.path.join(out_dir, stem + ".bin"), os.path.join(out_dir, stem + ".json")
    meta = {"file_name": os.path.basename(bin_path), "state_dict": {}}
    off = 0
    with open(bin_path, "wb", buffering=16 << 20) as f:
        for name, t in tensors.items():
            if not isinstance(t, torch.Tensor):
                continue
            if t.dtype not in _DTYPES:
                raise ValueError(f"{name}: unsupported dtype {t.dtype}")
            nbytes = t.element_size() * t.numel()
            meta["state_dict"][name] = {"dtype": _DTYPES[t.dtype], "shape": list(t.shape), "offset": off,
                                        "byte_size": nbytes}
            f.write(_raw_bytes(t))
            off += nbytes
    meta["total_byte_size"] = off
    with open(meta_path, "w") as f:
        json.dump(meta, f, indent=4)
    return meta_path


def shard_files(src_dir: str) -> List[str]:
    return sorted(os.path.join(src_dir, n) for n in os.listdir(src_dir) if n.endswith((".safetensors", ".pt")))


def convert_dir(src_dir: str, out_dir: str, workers: int = 4, partition: Optional[Tuple[int, int]] = None) -> List[str]:
    """Convert every shard of a directory (``partition=(i, n)`` takes shards i, i+n, ... so that several
    machines can split the work).  Non-tensor side files (config, tokenizer) are copied."""
    files = shard_files(src_dir)
    if partition is not None:
        i, n = partition
        files = files[i::n]
    os.makedirs(out_dir, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        metas = list(ex.map(lambda p: convert_shard(p, out_dir), files))
    for n in os.listdir(src_dir):
        if n.endswith((".json", ".jinja", ".txt", ".model")) and not os.path.exists(os.path.join(out_dir, n)):
            with open(os.path.join(src_dir, n), "rb") as a, open(os.path.join(out_dir, n), "wb") as b:
                b.write(a.read())
    return metas


def validate_dir(out_dir: str) -> int:
    """Check every metadata file against its .bin (sizes, contiguity, no overlap).  Returns #tensors."""
    n = 0
    for name in sorted(os.listdir(out_dir)):
        if not name.endswith(".json"):
            continue
        with open(os.path.join(out_dir, name)) as f:
            try:
                meta = json.load(f)
            except ValueError:
                continue
        if "state_dict" not in meta or "file_name" not in meta:
            continue
        size = os.path.getsize(os.path.join(out_dir, meta["file_name"]))
        if size != meta["total_byte_size"]:
            raise ValueError(f"{name}: .bin has {size} bytes, metadata says {meta['total_byte_size']}")
        end = 0
        for tname, e in meta["state_dict"].items():
            if e["offset"] != end:
                raise ValueError(f"{name}:{tname}: offset {e['offset']} != running end {end}")
            numel = 1
            for s in e["shape"]:
                numel *= s
            if e["dtype"] not in _FROM_STR:
                raise ValueError(f"{name}:{tname}: unknown dtype {e['dtype']}")
            esz = torch.empty(0, dtype=_FROM_STR[e["dtype"]]).element_size()
            if numel * esz != e["byte_size"]:
                raise ValueError(f"{name}:{tname}: shape and byte_size disagree")
            end += e["byte_size"]
            n += 1
    return n


class ConvertedCheckpoint:
    """Read-only view over a directory of converted shards (memory mapped)."""

    def __init__(self, out_dir: str):
        self.dir = out_dir
        self.index: Dict[str, Tuple[int, dict]] = {}
        self._maps: List[mmap.mmap] = []
        self._files = []
        for name in sorted(os.listdir(out_dir)):
            if not name.endswith(".json"):
                continue
            with open(os.path.join(out_dir, name)) as f:
                try:
                    meta = json.load(f)
                except ValueError:
                    continue
            if "state_dict" not in meta or "file_name" not in meta:
                continue
            path = os.path.join(out_dir, meta["file_name"])
            fh = open(path, "rb")
            self._files.append(fh)
            mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ) if meta["total_byte_size"] else None
            self._maps.append(mm)
            for tname, e in meta["state_dict"].items():
                self.index[tname] = (len(self._maps) - 1, e)

    def names(self) -> Iterable[str]:
        return self.index.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str) -> torch.Tensor:
        i, e = self.index[name]
        dt = _FROM_STR[e["dtype"]]
        if e["byte_size"] == 0:
            return torch.empty(e["shape"], dtype=dt)
        buf = memoryview(self._maps[i])[e["offset"]: e["offset"] + e["byte_size"]]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # read-only mapping: tensors are never written
            return torch.frombuffer(buf, dtype=torch.uint8).view(dt).view(*e["shape"])

    def total_bytes(self) -> int:
        return sum(e["byte_size"] for _, e in self.index.values())

    def loader(self) -> Callable[[str, Tuple[int, ...]], Optional[torch.Tensor]]:
        """Adapter for ``WeightSource(loader=...)``: full-precision tensor by checkpoint name, or None
        if the checkpoint lacks it.  Block-scaled FP8 weights are dequantised with their
        ``weight_scale_inv`` (128x128 blocks)."""
        def load(name: str, shape):
            if name not in self.index:
                return None
            t = self.get(name)
            if t.dtype == torch.float8_e4m3fn:
                sname = name.replace(".weight", ".weight_scale_inv")
                if sname in self.index:
                    from ..ops import ref
                    return ref.dequant_block(t, self.get(sname).float(), 128)
            return t.float()
        return load

    def close(self) -> None:
        for m in self._maps:
            if m is not None:
                try:
                    m.close()
                except BufferError:
                    pass          # tensors handed out still reference the mapping
        for f in self._files:
            f.close()


def save_model_checkpoint(cfg, src, path: str, shard_layers: int = 1) -> List[str]:
    """Write a model's full tensors (from a ``WeightSource``) as HF-named ``.pt`` shards — used by tests and
    to materialise synthetic checkpoints."""
    from ..models.weights import checkpoint_tensor_specs
    os.makedirs(path, exist_ok=True)
    shards: Dict[int, Dict[str, torch.Tensor]] = {}
    for name, shape, kind, layer in checkpoint_tensor_specs(cfg):
        shards.setdefault((layer + 1) // max(1, shard_layers), {})[name] = src.get(name, shape, kind).cpu()
    out = []
    for i, tensors in sorted(shards.items()):
        p = os.path.join(path, f"model-{i:05d}.pt")
        torch.save(tensors, p)
        out.append(p)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="convert .safetensors/.pt shards to .bin + .json")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--workers", type=int, default=4)
    ap.add_argument("--partition", default="", help="i/n: convert shards i, i+n, ...")
    ap.add_argument("--validate", action="store_true")
    a = ap.parse_args(argv)
    part = tuple(int(x) for x in a.partition.split("/")) if a.partition else None
    metas = convert_dir(a.src, a.dst, a.workers, part)
    print(f"converted {len(metas)} shard(s) into {a.dst}")
    if a.validate:
        print(f"validated {validate_dir(a.dst)} tensors")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
