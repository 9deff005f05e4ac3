"""Checkpoint tensor names of families whose published checkpoints do not use the DeepSeek-style names the weight
builder asks for.  ``aliased_loader`` wraps a loader (name, shape -> tensor or None) so that a miss on the builder's
name is retried under the family's own names.

Reference parity: the per-family parameter servers that map checkpoint names to module slots
(batchgen/models/mixtral/mixtral_parameter_server.py, batchgen/models/Qwen_Initializer.py).
"""
from __future__ import annotations

import re
from typing import Callable, List, Optional, Tuple

from ..config import ModelConfig

_MIXTRAL_PROJ = {"gate_proj": "w1", "down_proj": "w2", "up_proj": "w3"}


def candidates(cfg: ModelConfig, name: str) -> List[str]:
    """Other names ``name`` may carry in a published checkpoint of ``cfg``'s family (most likely first)."""
    out: List[str] = []
    if cfg.family == "mixtral":
        m = re.match(r"(model\.layers\.\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$", name)
        if m:
            out.append(f"{m.group(1)}.block_sparse_moe.experts.{m.group(2)}.{_MIXTRAL_PROJ[m.group(3)]}.weight")
        m = re.match(r"(model\.layers\.\d+)\.mlp\.gate\.weight$", name)
        if m:
            out.append(f"{m.group(1)}.block_sparse_moe.gate.weight")
    elif cfg.family == "qwen2_moe":
        if ".mlp.shared_experts." in name:
            out.append(name.replace(".mlp.shared_experts.", ".mlp.shared_expert."))
    return out


def aliased_loader(cfg: ModelConfig, loader: Callable[[str, Tuple[int, ...]], Optional[object]]):
    def load(name, shape):
        t = loader(name, shape)
        if t is not None:
            return t
        for alt in candidates(cfg, name):
            t = loader(alt, shape)
            if t is not None:
                return t
        return None
    return load
