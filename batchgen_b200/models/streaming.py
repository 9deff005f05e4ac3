"""Host-resident expert weights streamed through the GPU weight ring.

When the routed experts do not fit in HBM (Kimi-K3-shape models on one box) they stay in pinned host memory
and only a few layers' worth of slots exist on the GPU.  ``StreamedExperts`` registers every MoE layer's
stacked expert tensors as one ring module, installs the layer order as the copy queue, and lets the native
producer thread run ahead of the model: ``get(layer)`` blocks only if the copy has not landed yet and returns
an ``ExpertWeights`` whose tensors view the slot; ``release(layer)`` hands the slot back once the kernels
that read it (ordered on the current stream) are done.  A forward pass is one weight pass of the ring.

The quantised layouts are prepared once on the host (gate/up interleave for the fused SiLU epilogue), so a
slot is usable the moment it lands.  CUDA graphs cannot contain the host-side waits; streamed models run
the MoE part eagerly.

Reference parity: batchgen/models/wrappers/expert.py:127-172 (load / apply / free per expert module),
core/GPU_Weight_Buffer/GPU_Weight_Buffer.h:53-245 (ring, passes), core/HtoD_Engine/HtoD_Engine.cu:1016
(producer thread); batchgen/moe/streamed_sp8_mxfp4.py (streamed experts under EP).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..core.native import WeightRing
from ..ops.moe import ExpertWeights

_FIELDS = ("w13", "w2", "w13_s", "w2_s")


class StreamedExperts:
    def __init__(self, layers: Dict[int, ExpertWeights], device, num_slots: int = 3):
        self.device = torch.device(device)
        self.meta: Dict[int, ExpertWeights] = {}
        host: Dict[int, Dict[str, torch.Tensor]] = {}
        slot_bytes = 0
        pin = self.device.type == "cuda"
        for l, ew in layers.items():
            ew = ew.to_device_layout(force=True)
            ts = {}
            for f in _FIELDS:
                t = getattr(ew, f)
                if t is not None:
                    t = t.detach().to("cpu").contiguous()
                    ts[f] = t.pin_memory() if pin else t
            host[l] = ts
            # every tensor starts on a 256-byte boundary inside the slot
            slot_bytes = max(slot_bytes, sum((t.numel() * t.element_size() + 255) // 256 * 256 for t in ts.values()))
            self.meta[l] = ExpertWeights(w13=None, w2=None, quant=ew.quant, interleaved=ew.interleaved,
                                         activation=ew.activation)
        self.order = sorted(host)
        self.ring = WeightRing(num_slots, slot_bytes + 4096, str(self.device))
        for l in self.order:
            self.ring.register(self._key(l), host[l])
        self.ring.install_queue([self._key(l) for l in self.order])
        self.ring.start()
        self.bytes_per_pass = sum(t.numel() * t.element_size() for ts in host.values() for t in ts.values())
        self._open = False

    @staticmethod
    def _key(l: int) -> str:
        return f"routed_experts_{l}"

    def begin_step(self) -> None:
        if not self._open:
            self.ring.begin_pass()
            self._open = True

    def get(self, l: int, timeout_ms: int = 300_000) -> ExpertWeights:
        self.begin_step()
        ts = self.ring.get(self._key(l), timeout_ms)
        if ts is None:
            raise TimeoutError(f"streamed experts of layer {l} did not arrive within {timeout_ms} ms")
        m = self.meta[l]
        return ExpertWeights(w13=ts["w13"], w2=ts["w2"], w13_s=ts.get("w13_s"), w2_s=ts.get("w2_s"), quant=m.quant,
                             interleaved=m.interleaved, activation=m.activation)

    def release(self, l: int) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream if self.device.type == "cuda" else None
        self.ring.release(self._key(l), stream)

    def end_step(self) -> None:
        if self._open:
            self.ring.end_pass()
            self._open = False

    def stats(self) -> Dict[str, int]:
        return self.ring.stats()

    def close(self) -> None:
        self.ring.stop()
        self.ring.close()
