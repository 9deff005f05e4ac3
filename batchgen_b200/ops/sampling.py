"""Token sampling (greedy fast path, per-row temperature / top-k / top-p)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _ext, ref

_BAD_ROWS = {}


def bad_row_counter(device) -> torch.Tensor:
    """Device counter of rows whose logits had a non-finite maximum (never read on the hot path)."""
    key = str(device)
    if key not in _BAD_ROWS:
        _BAD_ROWS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _BAD_ROWS[key]


def greedy(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return sample(logits, None, None, None, None, out)


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], uniform: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """logits [T, V] (fp32 or bf16) -> int32 tokens [T].  ``temperature is None`` or a row with
    temperature <= 0 is greedy.  ``uniform`` ([T] in [0, 1)) is drawn here when omitted."""
    T, V = logits.shape
    if not logits.is_cuda:
        if temperature is None:
            tok = logits.float().argmax(-1)
        else:
            tk = top_k if top_k is not None else torch.zeros(T, dtype=torch.int64)
            tp = top_p if top_p is not None else torch.ones(T)
            tok = ref.sample(logits, temperature, tk.long(), tp, generator, uniform)
        tok = tok.to(torch.int32)
        if out is not None:
            out.copy_(tok)
            return out
        return tok
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    if out is None:
        out = torch.empty(T, dtype=torch.int32, device=logits.device)
    if temperature is not None and uniform is None:
        uniform = torch.rand(T, device=logits.device, generator=generator)
    rc = _ext.lib().bg_sample(ctypes.c_int(0 if logits.dtype == torch.float32 else 1), _ext.ptr(logits),
                              ctypes.c_longlong(logits.stride(0)), ctypes.c_int(T), ctypes.c_int(V),
                              _ext.ptr(temperature), _ext.ptr(top_k), _ext.ptr(top_p), _ext.ptr(uniform),
                              _ext.ptr(out), _ext.ptr(bad_row_counter(logits.device)), _ext.stream())
    _ext.check(rc, "bg_sample")
    return out
