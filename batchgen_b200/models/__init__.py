"""Model families.  ``build_model`` creates a ``Transformer`` for any registered config."""
from __future__ import annotations

from typing import Optional

import torch

from ..config import ModelConfig, get_model_config
from .transformer import AttnMeta, Transformer
from .weights import ParallelLayout, WeightSource, build_weights

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def build_model(cfg: ModelConfig, device="cpu", dtype="fp32", seed: int = 0, layout: Optional[ParallelLayout] = None,
                comm=None, max_positions: int = 8192, alias_experts_every: int = 0, loader=None,
                gen_device=None) -> Transformer:
    """Random-init (or ``loader``-fed) model on ``device``.  The registry role of the reference's
    get_initializer / get_parallel_strategy_manager (batchgen/get_initializer.py:19-46)."""
    dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    layout = layout or ParallelLayout()
    src = WeightSource(seed=seed, device=device, loader=loader, gen_device=gen_device)
    w = build_weights(cfg, layout, src, dt, alias_experts_every=alias_experts_every)
    return Transformer(cfg, w, layout, comm, max_positions)
