"""Kimi Delta Attention (KDA): gated delta-rule linear attention with a width-4 causal depthwise convolution
on q, k, v, L2-normalised q / k, a per-channel decay gate and a sigmoid-gated RMSNorm on the output.

``kda_forward`` serves prefill (packed sequences, optional continuation from a stored state) and decode (one
token per sequence) alike.  On CUDA it launches ``csrc/kda.cu``; on CPU (and as the oracle of the tests) it
runs the recurrence in fp32.  State lives in two pools indexed by a sequence's state slot:

    conv_state [slots, 3 * H * D, 3] fp32   the last three raw inputs of each q / k / v channel, oldest first
    rec_state  [slots, H, D, D]      fp32   S[key, value]

Reference parity: batchgen/models/moonshotai/kimi_linear/serving_modules.py:579-722 (projections and the
fused decode contract), :1074 (prefill), :1202 (decode); attention/kda_fused_decode.cu:147.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import _ext


@dataclass
class KDAParams:
    conv_w: torch.Tensor            # [3 * H * D, 4] fp32 (tap 3 multiplies the current token)
    conv_b: Optional[torch.Tensor]  # [3 * H * D] fp32 or None
    A_log: torch.Tensor             # [H] fp32
    dt_bias: torch.Tensor           # [H * D] fp32
    norm_w: torch.Tensor            # [D] fp32


def causal_conv1d_ref(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], window: torch.Tensor):
    """x [n, C] one sequence, w [C, 4], window [C, 3] (previous raw inputs, oldest first) ->
    (silu(conv) [n, C], new window [C, 3]).  fp32."""
    full = torch.cat([window.t().float(), x.float()], 0)               # [n + 3, C]
    n = x.shape[0]
    y = sum(full[i:i + n] * w[:, i].float() for i in range(4))
    if b is not None:
        y = y + b.float()
    return F.silu(y), full[-3:].t().contiguous()


def kda_gate(f: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, H: int, D: int) -> torch.Tensor:
    """Log decay per token, head and key channel: -exp(A_log[h]) * softplus(f + dt_bias)  (<= 0)."""
    return -A_log.float().exp().view(1, H, 1) * F.softplus(f.float().view(-1, H, D) + dt_bias.float().view(1, H, D))


def kda_recurrent_ref(q, k, v, g, beta, S, scale: float):
    """One sequence, fp32.  q, k, v, g [n, H, D]; beta [n, H] (after sigmoid); S [H, D, D] updated in place.
    Returns o [n, H, D]."""
    n = q.shape[0]
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    out = torch.empty_like(v)
    for t in range(n):
        S.mul_(g[t].exp().unsqueeze(-1))
        u = beta[t].unsqueeze(-1) * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S.add_(k[t].unsqueeze(-1) * u.unsqueeze(-2))
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def _forward_ref(qkv, f, beta, z, p: KDAParams, conv_state, rec_state, slots, cu, has_initial, H, D, scale, eps):
    T = qkv.shape[0]
    HD = H * D
    out = torch.zeros(T, HD, dtype=torch.float32, device=qkv.device)
    for i, slot in enumerate(slots):
        if slot < 0:
            continue
        a, b = cu[i], cu[i + 1]
        if b <= a:
            continue
        if has_initial is not None and not has_initial[i]:
            conv_state[slot].zero_()
            rec_state[slot].zero_()
        y, win = causal_conv1d_ref(qkv[a:b, : 3 * HD], p.conv_w, p.conv_b, conv_state[slot])
        conv_state[slot].copy_(win)
        qh, kh, vh = (y[:, s * HD:(s + 1) * HD].view(-1, H, D) for s in range(3))
        g = kda_gate(f[a:b], p.A_log, p.dt_bias, H, D)
        S = rec_state[slot].float()
        o = kda_recurrent_ref(qh, kh, vh, g, torch.sigmoid(beta[a:b].float()), S, scale)
        rec_state[slot].copy_(S)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * p.norm_w.float()
        out[a:b] = (o * torch.sigmoid(z[a:b].float().view(-1, H, D))).reshape(-1, HD)
    return out.to(qkv.dtype)


def kda_forward(qkv: torch.Tensor, f: torch.Tensor, beta: torch.Tensor, z: torch.Tensor, p: KDAParams,
                conv_state: torch.Tensor, rec_state: torch.Tensor, slots, cu_seqlens: Optional[Sequence[int]],
                has_initial: Optional[Sequence[int]], H: int, D: int, scale: float, eps: float) -> torch.Tensor:
    """qkv [T, >= 3HD] (raw q | k | v, may be a column view), f / z [T, HD], beta [T, >= H] (views allowed; unit
    column stride).  ``slots``: int32 tensor (or list) [nseq], < 0 skips; ``cu_seqlens`` None = one token per
    sequence; ``has_initial`` None = continue from the stored state.  Returns [T, HD] in qkv's dtype and
    updates both pools."""
    nseq = len(slots)
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16:
        sl = slots.tolist() if isinstance(slots, torch.Tensor) else list(slots)
        cu = list(range(nseq + 1)) if cu_seqlens is None else list(cu_seqlens)
        return _forward_ref(qkv, f, beta, z, p, conv_state, rec_state, sl, cu, has_initial, H, D, scale, eps)
    dev = qkv.device
    for t in (qkv, f, beta, z):
        assert t.stride(1) == 1
    if not isinstance(slots, torch.Tensor):
        slots = torch.tensor(list(slots), dtype=torch.int32, device=dev)
    cu_t = None if cu_seqlens is None else (
        cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(list(cu_seqlens), dtype=torch.int32, device=dev))
    hi_t = None if has_initial is None else (
        has_initial if isinstance(has_initial, torch.Tensor) else torch.tensor([int(x) for x in has_initial], dtype=torch.int32, device=dev))
    out = torch.empty(qkv.shape[0], H * D, dtype=torch.bfloat16, device=dev)
    rc = _ext.lib().bg_kda_forward(
        _ext.ptr(qkv), ctypes.c_int(qkv.stride(0)), _ext.ptr(f), ctypes.c_int(f.stride(0)), _ext.ptr(beta),
        ctypes.c_int(beta.stride(0)), _ext.ptr(z), ctypes.c_int(z.stride(0)), _ext.ptr(p.conv_w), _ext.ptr(p.conv_b),
        _ext.ptr(p.A_log), _ext.ptr(p.dt_bias), _ext.ptr(p.norm_w), _ext.ptr(conv_state), _ext.ptr(rec_state),
        _ext.ptr(cu_t), _ext.ptr(slots), _ext.ptr(hi_t), _ext.ptr(out), ctypes.c_int(nseq), ctypes.c_int(H),
        ctypes.c_int(D), ctypes.c_float(scale), ctypes.c_float(eps), _ext.stream())
    _ext.check(rc, "bg_kda_forward")
    return out
