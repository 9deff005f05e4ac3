"""Device-resident per-row sampling parameters for the decode loop.

Building the ``[B]`` temperature / top-p / top-k tensors from Python lists on every step costs a pageable
host->device copy that cannot retire before the graph replay queued ahead of it, so the host would stand
still inside a parameter upload.  ``DecodeSamplingResidency`` keeps the three tensors on the device and
rewrites them (from pinned staging, asynchronously) only when the ordered row set changes.  In the steady
state a step does three comparisons and three slices: no allocation, no copy, no readback.

Staleness would be silent (a wrong temperature still yields plausible tokens), so the cache key is strict:
the composition epoch of the batch, the row-order epoch, and the identity of the rows list, which callers
rebind (never mutate) whenever rows change.  Length disagreement and unresolved rows fail loudly;
``verify=True`` recomputes and compares on every call.

Reference parity: batchgen/worker/sampling_residency.py:1-120 (contract), :289 (DecodeSamplingResidency);
batchgen/sampling.py:51-100 (host-decided greedy / sampled split without a device sync).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch


class SamplingResidencyShapeError(RuntimeError):
    pass


class SamplingResidencyRowError(RuntimeError):
    pass


@dataclass(frozen=True)
class ResidentSamplingView:
    temperature: torch.Tensor      # [n] float32
    top_p: torch.Tensor            # [n] float32
    top_k: torch.Tensor            # [n] int32
    all_greedy: bool               # decided on the host: the sampler can take its argmax path without a sync
    any_top_k: bool
    any_top_p: bool


def _row_values(params: Any) -> Tuple[float, float, int]:
    if params is None:
        raise SamplingResidencyRowError("a decode row resolved to no sampling parameters")
    get = params.get if isinstance(params, dict) else lambda k, d=None: getattr(params, k, d)
    t = float(get("temperature", 1.0) if get("temperature", 1.0) is not None else 1.0)
    p = float(get("top_p", 1.0) if get("top_p", 1.0) is not None else 1.0)
    k = int(get("top_k", 0) or 0)
    return t, p, max(k, 0)


class DecodeSamplingResidency:
    def __init__(self, max_rows: int, device, verify: bool = False):
        self.device = torch.device(device)
        self.max_rows, self.verify = max_rows, verify
        pin = self.device.type == "cuda"
        self._t = torch.ones(max_rows, dtype=torch.float32, device=self.device)
        self._p = torch.ones(max_rows, dtype=torch.float32, device=self.device)
        self._k = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self._ht = torch.ones(max_rows, dtype=torch.float32, pin_memory=pin)
        self._hp = torch.ones(max_rows, dtype=torch.float32, pin_memory=pin)
        self._hk = torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin)
        self._key: Optional[Tuple[int, int, int]] = None
        self._rows_obj: Optional[Sequence] = None
        self._n = 0
        self._flags = (True, False, False)
        self.uploads = 0
        self.hits = 0

    def _compute(self, row_params: Sequence[Any]) -> Tuple[List[float], List[float], List[int]]:
        ts, ps, ks = [], [], []
        for prm in row_params:
            t, p, k = _row_values(prm)
            ts.append(t); ps.append(p); ks.append(k)
        return ts, ps, ks

    def view(self, rows: Sequence, row_params: Sequence[Any], composition_epoch: int, row_epoch: int
             ) -> ResidentSamplingView:
        """``rows``: the decode row list (rebound on every change); ``row_params[i]``: sampling parameters of
        row i (dict or object with temperature / top_p / top_k)."""
        n = len(rows)
        if len(row_params) != n:
            raise SamplingResidencyShapeError(f"{n} rows but {len(row_params)} parameter sets")
        if n > self.max_rows:
            raise SamplingResidencyShapeError(f"{n} rows exceed the resident capacity {self.max_rows}")
        key = (composition_epoch, row_epoch, n)
        fresh = self._key != key or self._rows_obj is not rows
        if fresh:
            ts, ps, ks = self._compute(row_params)
            self._ht[:n] = torch.tensor(ts, dtype=torch.float32)
            self._hp[:n] = torch.tensor(ps, dtype=torch.float32)
            self._hk[:n] = torch.tensor(ks, dtype=torch.int32)
            self._t[:n].copy_(self._ht[:n], non_blocking=True)
            self._p[:n].copy_(self._hp[:n], non_blocking=True)
            self._k[:n].copy_(self._hk[:n], non_blocking=True)
            self._flags = (all(t <= 0.0 for t in ts), any(k > 0 for k in ks), any(p < 1.0 for p in ps))
            self._key, self._rows_obj, self._n = key, rows, n
            self.uploads += 1
        else:
            self.hits += 1
            if self.verify:
                ts, ps, ks = self._compute(row_params)
                if self._ht[:n].tolist() != [float(torch.tensor(t, dtype=torch.float32)) for t in ts] \
                        or self._hk[:n].tolist() != ks:
                    raise SamplingResidencyRowError("resident sampling parameters are stale for this row order")
        return ResidentSamplingView(self._t[:n], self._p[:n], self._k[:n], *self._flags)

    def invalidate(self) -> None:
        self._key, self._rows_obj = None, None
