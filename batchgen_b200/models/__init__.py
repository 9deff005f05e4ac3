"""Model families.  ``build_model`` creates a ``Transformer`` (or, for DeepSeek-V4, a ``DeepSeekV4``) for any
registered config."""
from __future__ import annotations

from typing import Optional

import torch

from ..config import ModelConfig, get_model_config
from .transformer import AttnMeta, Transformer
from .weights import ParallelLayout, WeightSource, build_weights

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def build_model(cfg: ModelConfig, device="cpu", dtype="fp32", seed: int = 0, layout: Optional[ParallelLayout] = None,
                comm=None, max_positions: int = 8192, alias_experts_every: int = 0, loader=None,
                gen_device=None, stream_experts: bool = False, ring_slots: int = 3) -> Transformer:
    """Random-init (or ``loader``-fed) model on ``device``.  The registry role of the reference's
    get_initializer / get_parallel_strategy_manager (batchgen/get_initializer.py:19-46)."""
    dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    layout = layout or ParallelLayout()
    if loader is not None:
        from .checkpoint_names import aliased_loader
        loader = aliased_loader(cfg, loader)            # published names of the family, when they differ
    src = WeightSource(seed=seed, device=device, loader=loader, gen_device=gen_device)
    if cfg.is_v4:
        from .deepseek_v4 import DeepSeekV4, build_v4_weights
        return DeepSeekV4(cfg, build_v4_weights(cfg, layout, src, dt), layout, comm, max_positions)
    w = build_weights(cfg, layout, src, dt, alias_experts_every=alias_experts_every,
                      experts_on_host=stream_experts)
    model = Transformer(cfg, w, layout, comm, max_positions)
    if stream_experts:
        # routed experts stay in (pinned) host memory and flow through the native weight ring
        from .streaming import StreamedExperts
        layers = {l: lw.experts for l, lw in enumerate(w.layers) if lw.experts is not None}
        model.streamer = StreamedExperts(layers, device, num_slots=ring_slots)
        for lw in w.layers:
            lw.experts = None
    return model
