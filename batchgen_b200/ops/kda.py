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


def kda_chunk_ref(q, k, v, g, beta, S, scale: float, chunk: int = 64):
    """The same recurrence in chunk form (the shape a tensor-core prefill kernel takes): inside a chunk the
    writes u_i = beta_i (v_i - S_(i-1)'^T k_i) solve a unit lower-triangular system, after which outputs and the
    state at the chunk end are plain matrix products.  With G the running sum of the log decay inside the chunk,

        M[i, j]  = sum_c k_i[c] k_j[c] exp(G_i[c] - G_j[c])          (j < i)
        (I + diag(beta) M) U = diag(beta) (V - (K * exp(G)) S_0)
        O        = (Q * exp(G)) S_0 + tril(Q-to-K decayed products) U
        S_end    = exp(G_last) * S_0 + sum_j (k_j * exp(G_last - G_j)) u_j^T

    q, k, v, g [n, H, D]; beta [n, H] (after sigmoid); S [H, D, D] updated in place; returns o [n, H, D].  fp32."""
    n, H, D = q.shape
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    out = torch.empty_like(v)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        C = b - a
        qc, kc, vc, bc = (t[a:b].transpose(0, 1) for t in (q, k, v, beta.unsqueeze(-1)))     # [H, C, D] / [H, C, 1]
        G = g[a:b].transpose(0, 1).cumsum(1)                                               # [H, C, D]
        # decayed pair products; the exponent is <= 0 wherever it is used (j <= i)
        diff = (G.unsqueeze(2) - G.unsqueeze(1)).clamp_max(0.0).exp()                       # [H, i, j, D]
        kk = torch.einsum("hid,hjd,hijd->hij", kc, kc, diff)
        qk = torch.einsum("hid,hjd,hijd->hij", qc, kc, diff)
        eye = torch.eye(C, dtype=q.dtype, device=q.device)
        A = eye + bc * torch.tril(kk, -1)
        rhs = bc * (vc - torch.einsum("hcd,hdv->hcv", kc * G.exp(), S))
        U = torch.linalg.solve_triangular(A, rhs, upper=False)
        out[a:b] = (torch.einsum("hcd,hdv->hcv", qc * G.exp(), S) + torch.tril(qk) @ U).transpose(0, 1)
        last = G[:, -1:, :]                                                                 # [H, 1, D]
        S.mul_(last.squeeze(1).exp().unsqueeze(-1))
        S.add_(torch.einsum("hcd,hcv->hdv", kc * (last - G).exp(), U))
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
        step = kda_chunk_ref if (b - a) > 128 else kda_recurrent_ref           # long prompts: chunk form
        o = step(qh, kh, vh, g, torch.sigmoid(beta[a:b].float()), S, scale)
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
