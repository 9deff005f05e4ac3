"""batchgen_b200 — a Blackwell (B200, sm_100a) native batch-inference engine.

The package is organised in layers:

``config``      model / engine dataclasses and the named presets
``ops``         hot operators: hand-written sm_100a CUDA kernels with fp32 torch
                reference implementations used on CPU and as numerics oracles
``models``      model families (DeepSeek-V3/R1, GLM-5.x DSA, Kimi-K3 MXFP4, GQA families)
``parallel``    symmetric heap over NVLink, fused compute+collective kernels,
                NCCL baselines
``runtime``     sequence state machine, paged KV, schedulers, engine, CUDA graphs
``core``        native (C++) weight ring, host paged KV, prefix cache coordinator
``server``      OpenAI-style file/batch HTTP server, control plane and client
``ckpt``        checkpoint converter (``.bin`` + ``.json`` shard format)
``utils``       event log, timers, memfd helpers
"""

__version__ = "0.1.0"

from .config import EngineConfig, ModelConfig, get_model_config  # noqa: F401
