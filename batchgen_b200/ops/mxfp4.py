"""MXFP4 (e2m1 values, one e8m0 scale per 32) expert weights: GEMMs and conversion.

On CUDA the GEMMs run ``gemm_mxfp4.cu``: packed weights go from HBM to shared memory as 4-bit data and are
expanded to bf16 inside the CTA, then multiplied on tcgen05 with fp32 accumulation.  On CPU the same
contract is met by dequantising and multiplying in fp32.

Reference parity: quantiser / layout batchgen/quantization/mxfp4.py:30 and
batchgen/models/moonshotai/kimi_linear/k3/mxfp4_layout.py:37-38,179-182; grouped GEMMs
batchgen_kernels/src/moe/mxfp4/marlin_grouped_gemm.cu and batchgen/moe/fused_moe_mxfp4_resident.py:946-1125.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _ext, ref

EPI_STORE, EPI_SILU_MUL = 0, 1


def quantize(w: torch.Tensor):
    """[..., N, K] float -> (packed uint8 [..., N, K/2], scales uint8 [..., N, K/32])."""
    lead = w.shape[:-2]
    N, K = w.shape[-2:]
    q, s = ref.mxfp4_quant(w.reshape(-1, K))
    return q.view(*lead, N, K // 2), s.view(*lead, N, K // 32)


def dequantize(wq: torch.Tensor, ws: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Expand packed weights to ``dtype`` (exact: every MXFP4 value is representable in bf16)."""
    lead = wq.shape[:-1]
    K = wq.shape[-1] * 2
    if not wq.is_cuda:
        return ref.mxfp4_dequant(wq.reshape(-1, K // 2), ws.reshape(-1, K // 32)).view(*lead, K).to(dtype)
    wq = wq.contiguous()
    ws = ws.contiguous()
    out = torch.empty(*lead, K, dtype=torch.bfloat16, device=wq.device)
    rc = _ext.lib().bg_mxfp4_dequant(_ext.ptr(wq), _ext.ptr(ws), _ext.ptr(out), ctypes.c_longlong(out.numel()),
                                     _ext.stream())
    _ext.check(rc, "bg_mxfp4_dequant")
    return out.to(dtype)


def _launch(epi, x, wq2d, ws2d, out, offsets, groups, M, N, K):
    rc = _ext.lib().bg_mxfp4_gemm(
        ctypes.c_int(epi), _ext.ptr(x), _ext.ptr(wq2d), _ext.ptr(ws2d), _ext.ptr(out), ctypes.c_int(out.stride(0)),
        _ext.ptr(offsets), ctypes.c_int(groups), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(_ext.num_sms(x.device)), _ext.ptr(_ext.status_word(x.device)), _ext.stream())
    _ext.check(rc, "bg_mxfp4_gemm")


def mxfp4_gemm(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, K] bf16 x MXFP4 [N, K] -> [T, N] bf16."""
    N, K = wq.shape[0], wq.shape[1] * 2
    if not x.is_cuda:
        return (x.float() @ dequantize(wq, ws, torch.float32).t()).to(x.dtype)
    T = x.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    if T:
        _launch(EPI_STORE, x.contiguous(), wq, ws, out, None, 1, T, N, K)
    return out


def grouped_mxfp4_gemm(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, offsets: torch.Tensor,
                       silu_mul: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ragged grouped GEMM over rows grouped by expert (segment e = offsets[e]:offsets[e+1], starts
    128-aligned on the GPU path).  wq [E, N, K/2], ws [E, N, K/32].  ``silu_mul``: the rows of each expert
    are stored gate/up interleaved in blocks of 32 and the output is silu(gate) * up with N/2 columns."""
    E, N, Kh = wq.shape
    K = Kh * 2
    R = x.shape[0]
    if not x.is_cuda:
        from .gemm import interleave_gate_up_rows
        y = torch.zeros(R, N, dtype=torch.float32)
        off = offsets.tolist()
        w = dequantize(wq, ws, torch.float32)
        for e in range(E):
            a, b = off[e], off[e + 1]
            if b > a:
                y[a:b] = x[a:b].float() @ w[e].t()
        if silu_mul:
            inv = torch.argsort(interleave_gate_up_rows(N))
            y = ref.silu_mul(y[:, inv])
        return y.to(x.dtype)
    n_out = N // 2 if silu_mul else N
    if out is None:
        out = torch.empty(R, n_out, dtype=torch.bfloat16, device=x.device)
    if R:
        assert offsets.dtype == torch.int32 and offsets.is_cuda
        _launch(EPI_SILU_MUL if silu_mul else EPI_STORE, x.contiguous(), wq.view(E * N, Kh), ws.view(E * N, K // 32),
                out, offsets, E, R, N, K)
    return out
