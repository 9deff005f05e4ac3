"""Fused normalisation / quantisation / RoPE / latent-KV-write operators.

Every function accepts CPU tensors (fp32 reference path) or CUDA bf16 tensors (sm_100a kernels in
``csrc/elementwise.cu``).  Quantised activations are returned as ``(q, s)`` where ``s`` is logically
``[T, K/128]`` but, on the GPU, physically stored block-major (``s.stride(0) == 1``) — the layout
the tcgen05 GEMM epilogue reads with coalesced loads.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _ext, ref

FP8 = torch.float8_e4m3fn


def _scale_buffer(T: int, KB: int, device) -> torch.Tensor:
    """Logical [T, KB] view over a [KB, T4] buffer (T padded to 4 for 16-byte row alignment)."""
    tp = (T + 3) // 4 * 4
    return torch.empty(KB, tp, dtype=torch.float32, device=device).t()[:T]


def act_quant(x: torch.Tensor, pow2_scale: bool = False, silu_mul: bool = False,
              valid_rows: Optional[torch.Tensor] = None,
              row_src: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """1x128 e4m3 quantisation of x [T, K] (or of silu(x[:, :K]) * x[:, K:] when ``silu_mul``).
    ``valid_rows`` (device int) bounds the rows processed; ``row_src`` (int32 [T]) marks padding rows of
    expert segments with a negative value: they are skipped (their outputs stay undefined)."""
    if not x.is_cuda:
        y = ref.silu_mul(x) if silu_mul else x
        return ref.act_quant(y, 128, pow2_scale)
    T = x.shape[0]
    K = x.shape[1] // 2 if silu_mul else x.shape[1]
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = _scale_buffer(T, K // 128, x.device)
    rc = _ext.lib().bg_act_quant(ctypes.c_int(1 if silu_mul else 0), _ext.ptr(x), _ext.ptr(q), _ext.ptr(s),
                                 ctypes.c_int(s.stride(1)), ctypes.c_int(T), ctypes.c_int(K),
                                 ctypes.c_int(x.stride(0)), ctypes.c_int(int(pow2_scale)), _ext.ptr(valid_rows),
                                 _ext.ptr(row_src), _ext.stream())
    _ext.check(rc, "bg_act_quant")
    return q, s


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
            quant: bool = False, want_bf16: bool = True, pow2_scale: bool = False):
    """(residual += x;) y = rmsnorm(residual or x) * w.

    Returns ``(y, q, s)``: ``y`` bf16/fp32 output (None if ``want_bf16`` is False on the GPU path),
    ``q``/``s`` the e4m3 quantisation of ``y`` (None unless ``quant``).  ``residual`` is updated in
    place and must be contiguous."""
    if not x.is_cuda:
        if residual is not None:
            residual.copy_((x.float() + residual.float()).to(residual.dtype))
            src = residual
        else:
            src = x
        y = ref.rmsnorm(src, w, eps)
        q = s = None
        if quant:
            q, s = ref.act_quant(y, 128, pow2_scale)
        return y, q, s
    T, H = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    y = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    q = s = None
    s_stride = 0
    if quant:
        q = torch.empty(T, H, dtype=FP8, device=x.device)
        s = _scale_buffer(T, H // 128, x.device)
        s_stride = s.stride(1)
    if residual is not None:
        assert residual.is_contiguous() and residual.dtype == torch.bfloat16
    rc = _ext.lib().bg_rmsnorm(_ext.ptr(x), _ext.ptr(residual), _ext.ptr(w), _ext.ptr(y), _ext.ptr(q), _ext.ptr(s),
                               ctypes.c_int(s_stride), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(x.stride(0)),
                               ctypes.c_int(H), ctypes.c_float(eps), ctypes.c_int(int(pow2_scale)), _ext.stream())
    _ext.check(rc, "bg_rmsnorm")
    return y, q, s


def mla_kv_write(kv_a: torch.Tensor, norm_w: torch.Tensor, positions: torch.Tensor, cos_table: torch.Tensor,
                 sin_table: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor, kv_lora: int,
                 eps: float, interleaved: bool) -> None:
    """cache[slot] = [rmsnorm(kv_a[:, :kv_lora]) * w | rope(kv_a[:, kv_lora:])]; slot < 0 skipped.
    cache: [P, page, kv_lora + rope]; cos/sin tables: [max_pos, rope/2] fp32."""
    rope = kv_a.shape[1] - kv_lora
    if not kv_a.is_cuda:
        cos, sin = cos_table[positions.long()], sin_table[positions.long()]
        rows = ref.mla_kv_prepare(kv_a, norm_w, cos, sin, kv_lora, eps, interleaved)
        ref.kv_cache_write(cache, rows, slot_mapping)
        return
    assert cache.dtype == torch.bfloat16 and cache.is_contiguous() and kv_a.stride(1) == 1
    assert positions.dtype == torch.int32 and slot_mapping.dtype == torch.int64
    rc = _ext.lib().bg_mla_kv_write(_ext.ptr(kv_a), ctypes.c_int(kv_a.stride(0)), _ext.ptr(norm_w),
                                    _ext.ptr(positions), _ext.ptr(cos_table), _ext.ptr(sin_table),
                                    _ext.ptr(slot_mapping), _ext.ptr(cache), ctypes.c_int(kv_a.shape[0]),
                                    ctypes.c_int(kv_lora), ctypes.c_int(rope), ctypes.c_float(eps),
                                    ctypes.c_int(int(interleaved)), _ext.stream())
    _ext.check(rc, "bg_mla_kv_write")


def rope_q_(q: torch.Tensor, positions: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
            rope: int, interleaved: bool) -> torch.Tensor:
    """In-place RoPE on the last ``rope`` dims of every head of q [T, H, D]."""
    if not q.is_cuda:
        cos, sin = cos_table[positions.long()], sin_table[positions.long()]
        q[..., -rope:] = ref.apply_rope(q[..., -rope:], cos, sin, interleaved)
        return q
    T, H, D = q.shape
    assert q.stride(2) == 1 and q.stride(1) == D and positions.dtype == torch.int32
    rc = _ext.lib().bg_rope_q(_ext.ptr(q), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(D), ctypes.c_int(rope),
                              _ext.ptr(positions), _ext.ptr(cos_table), _ext.ptr(sin_table),
                              ctypes.c_int(int(interleaved)), ctypes.c_longlong(q.stride(0)), _ext.stream())
    _ext.check(rc, "bg_rope_q")
    return q
