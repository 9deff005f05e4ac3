"""INT4 W4A16 expert weights (symmetric, group size 32, bf16 group scales): conversion and GEMMs.

Weights are stored two offset-binary nibbles per byte (value = q - 8, low nibble = even k) with one bf16
scale per 32 weights.  On CUDA the GEMMs run the 4-bit tcgen05 kernel of ``csrc/gemm_mxfp4.cu`` in its INT4
mode (weights stay 4-bit from HBM to shared memory, expanded to bf16 in the CTA); on CPU the contract is
met by dequantising and multiplying in fp32.

Reference parity: the Kimi-K2.5 family's INT4 W4A16 gs=32 experts (Marlin and INT4 WGMMA grouped kernels,
batchgen/models/moonshotai/kimi_k25/).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _ext, ref

GROUP = 32


def quantize(w: torch.Tensor):
    """[..., N, K] float -> (packed uint8 [..., N, K/2], scales bf16 [..., N, K/32])."""
    lead = w.shape[:-2]
    N, K = w.shape[-2:]
    assert K % GROUP == 0
    wf = w.float().reshape(-1, K // GROUP, GROUP)
    scale = (wf.abs().amax(-1) / 7.0).clamp_min(1e-8).to(torch.bfloat16)
    q = torch.clamp(torch.round(wf / scale.float().unsqueeze(-1)), -8, 7).to(torch.int16) + 8
    q = q.reshape(-1, K)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
    return packed.view(*lead, N, K // 2), scale.view(*lead, N, K // GROUP)


def dequantize(wq: torch.Tensor, ws: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    lead = wq.shape[:-1]
    K = wq.shape[-1] * 2
    q = wq.reshape(-1, K // 2)
    lo = (q & 0xF).to(torch.float32) - 8.0
    hi = (q >> 4).to(torch.float32) - 8.0
    w = torch.stack([lo, hi], -1).view(-1, K)
    s = ws.reshape(-1, K // GROUP).float().repeat_interleave(GROUP, 1)
    return (w * s).view(*lead, K).to(dtype)


def _launch(epi, x, wq2d, ws2d, out, offsets, groups, M, N, K):
    rc = _ext.lib().bg_int4_gemm(
        ctypes.c_int(epi), _ext.ptr(x), _ext.ptr(wq2d), _ext.ptr(ws2d), _ext.ptr(out), ctypes.c_int(out.stride(0)),
        _ext.ptr(offsets), ctypes.c_int(groups), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(_ext.num_sms(x.device)), _ext.ptr(_ext.status_word(x.device)), _ext.stream())
    _ext.check(rc, "bg_int4_gemm")


def int4_gemm(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    """[T, K] bf16 x INT4 [N, K] -> [T, N] bf16."""
    N, K = wq.shape[0], wq.shape[1] * 2
    if not x.is_cuda:
        return (x.float() @ dequantize(wq, ws).t()).to(x.dtype)
    out = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    if x.shape[0]:
        _launch(0, x.contiguous(), wq, ws.contiguous(), out, None, 1, x.shape[0], N, K)
    return out


def grouped_int4_gemm(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, offsets: torch.Tensor,
                      silu_mul: bool = False) -> torch.Tensor:
    """Ragged grouped GEMM (segment e = offsets[e]:offsets[e+1], 128-aligned starts on the GPU).  wq [E, N, K/2],
    ws [E, N, K/32] bf16.  ``silu_mul``: rows interleaved gate/up in blocks of 32, output silu(gate) * up."""
    E, N, Kh = wq.shape
    K = Kh * 2
    R = x.shape[0]
    if not x.is_cuda:
        from .gemm import interleave_gate_up_rows
        y = torch.zeros(R, N, dtype=torch.float32)
        off = offsets.tolist()
        w = dequantize(wq, ws)
        for e in range(E):
            a, b = off[e], off[e + 1]
            if b > a:
                y[a:b] = x[a:b].float() @ w[e].t()
        if silu_mul:
            y = ref.silu_mul(y[:, torch.argsort(interleave_gate_up_rows(N))])
        return y.to(x.dtype)
    out = torch.empty(R, N // 2 if silu_mul else N, dtype=torch.bfloat16, device=x.device)
    if R:
        _launch(1 if silu_mul else 0, x.contiguous(), wq.view(E * N, Kh), ws.contiguous().view(E * N, K // GROUP), out,
                offsets, E, R, N, K)
    return out
