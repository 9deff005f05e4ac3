"""Attention operators over the paged KV cache.

MLA runs in the *absorbed* form everywhere: the cache holds one latent row per token
(``[rmsnorm(c_kv) | rope(k_pe)]``, 576 wide for DeepSeek/GLM/Kimi), queries are projected into the
latent space (``q_nope @ W_UK``) and the attention output (latent width) is projected back with
``W_UV``.  Contract of the decode op follows batchgen/attention/mla/paged_decode.py:1-31, of the
sparse op batchgen/attention/mla/sparse_dispatch.py:4-20.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _ext, ref


def mla_decode(q_abs: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
               seqlens: torch.Tensor, scale: float, kv_lora: int) -> torch.Tensor:
    """q_abs [B, H, kv_lora], q_pe [B, H, rope], cache [P, page, kv_lora+rope], block_table [B, maxp]
    int32, seqlens [B] int32 -> latent output [B, H, kv_lora]."""
    if q_abs.is_cuda:
        from . import mla_cuda
        return mla_cuda.mla_decode(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora)
    return ref.mla_decode(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora)


def mla_prefill(q_abs: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                cu_seqlens: Sequence[int], ctx_lens: Sequence[int], scale: float, kv_lora: int) -> torch.Tensor:
    """Varlen causal absorbed MLA over the paged cache (new rows already written)."""
    if q_abs.is_cuda:
        from . import mla_cuda
        return mla_cuda.mla_prefill(q_abs, q_pe, cache, block_table, cu_seqlens, ctx_lens, scale, kv_lora)
    return ref.mla_prefill(q_abs, q_pe, cache, block_table, cu_seqlens, ctx_lens, scale, kv_lora)


def sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora):
    if q_abs.is_cuda:
        from . import mla_cuda
        return mla_cuda.sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora)
    return ref.sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora)


def _head_gemm(a: torch.Tensor, a_head: int, K: int, w: torch.Tensor, out: torch.Tensor, d_row: int, d_head: int):
    T, H, N = a.shape[0], w.shape[0], w.shape[1]
    rc = _ext.lib().bg_head_gemm(_ext.ptr(a), ctypes.c_longlong(a.stride(0)), ctypes.c_int(a_head),
                                 ctypes.c_longlong(a.stride(0)), _ext.ptr(w), _ext.ptr(out), ctypes.c_longlong(d_row),
                                 ctypes.c_longlong(d_head), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(N),
                                 ctypes.c_int(K), _ext.ptr(_ext.status_word(a.device)), _ext.stream())
    _ext.check(rc, "bg_head_gemm")


def mla_q_absorb(q: torch.Tensor, w_uk_t: torch.Tensor, nope: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, nope + rope] (the q projection, in place) x W_UK^T [H, kv_lora, nope] -> q_abs [T, H, kv_lora].
    ``out`` may be a [T, H, kv_lora] view of a wider buffer (unit inner stride)."""
    T, H, D = q.shape
    if (q.is_cuda and q.dtype == torch.bfloat16) and q.stride(2) == 1 and q.stride(1) == D and nope % 64 == 0 and D % 8 == 0:
        if out is None:
            out = torch.empty(T, H, w_uk_t.shape[1], dtype=q.dtype, device=q.device)
        _head_gemm(q.view(T, H * D) if q.is_contiguous() else q.as_strided((T, H * D), (q.stride(0), 1)), D, nope,
                   w_uk_t, out, out.stride(0), out.stride(1))
        return out
    if q.is_cuda:
        from .policy import library_fallback
        library_fallback("mla_q_absorb", f"q {tuple(q.shape)} {q.dtype} strides {q.stride()}, nope {nope}; the per-head "
                                         "GEMM needs bf16, dense heads, nope % 64 == 0")
    res = torch.bmm(q[..., :nope].transpose(0, 1), w_uk_t.transpose(1, 2)).transpose(0, 1)
    if out is not None:
        out.copy_(res)
        return out
    return res


def mla_out_absorb(o_lat: torch.Tensor, w_uv: torch.Tensor) -> torch.Tensor:
    """o_lat [T, H, kv_lora] x W_UV [H, v, kv_lora] -> [T, H * v]."""
    T, H, L = o_lat.shape
    V = w_uv.shape[1]
    if (o_lat.is_cuda and o_lat.dtype == torch.bfloat16) and o_lat.is_contiguous() and L % 64 == 0 and V % 8 == 0:
        out = torch.empty(T, H * V, dtype=o_lat.dtype, device=o_lat.device)
        _head_gemm(o_lat.view(T, H * L), L, L, w_uv, out, out.stride(0), V)
        return out
    if o_lat.is_cuda:
        from .policy import library_fallback
        library_fallback("mla_out_absorb", f"o_lat {tuple(o_lat.shape)} {o_lat.dtype}, v {V}; the per-head GEMM needs "
                                           "bf16, contiguous, latent % 64 == 0, v % 8 == 0")
    return torch.bmm(o_lat.transpose(0, 1), w_uv.transpose(1, 2)).transpose(0, 1).reshape(T, -1)


_GQA_SCRATCH = {}


def gqa_decode(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, seqlens: torch.Tensor, num_kv_heads: int,
               scale: float, window: int = 0, sinks: Optional[torch.Tensor] = None, num_splits: int = 0) -> torch.Tensor:
    """Paged GQA decode.  q [B, Hq, D]; cache [P, page, 2 * Hkv * D] (K heads then V heads per token);
    seqlens [B] int32 = tokens visible to each query (its own included) -> [B, Hq, D].  ``window`` > 0 limits
    every query to its last ``window`` positions; ``sinks`` [Hq] joins the softmax denominator."""
    B, Hq, D = q.shape
    page = cache.shape[1]
    if not (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128)):
        if q.is_cuda:
            from .policy import library_fallback
            library_fallback("gqa_decode", f"q {q.dtype}, head_dim {D}; the kernel needs bf16 and head_dim 64 or 128")
        out = torch.zeros_like(q)
        for b in range(B):
            L = int(seqlens[b])
            kv = ref.gather_paged(cache, block_table[b], L)
            ks = kv[:, : num_kv_heads * D].reshape(L, num_kv_heads, D)
            vs = kv[:, num_kv_heads * D:].reshape(L, num_kv_heads, D)
            out[b:b + 1] = ref.gqa_attention(q[b:b + 1], ks, vs, scale, q_start=L - 1, window=window, sinks=sinks)
        return out
    q = q.contiguous()
    if num_splits <= 0:
        ctas = B * num_kv_heads
        sms = _ext.num_sms(q.device)
        max_tiles = max(1, (block_table.shape[1] * page) // 64)
        if window > 0:
            max_tiles = min(max_tiles, window // 64 + 2)
        num_splits = max(1, min(16, -(-2 * sms // ctas), max_tiles))
    out = torch.empty_like(q)
    part_o = part_ml = None
    if num_splits > 1:
        key = (str(q.device), B * Hq * num_splits, D)
        buf = _GQA_SCRATCH.get(key)
        if buf is None:
            buf = (torch.empty(B * Hq * num_splits * D, dtype=torch.float32, device=q.device),
                   torch.empty(B * Hq * num_splits * 2, dtype=torch.float32, device=q.device))
            _GQA_SCRATCH[key] = buf
        part_o, part_ml = buf
    rc = _ext.lib().bg_gqa_decode(_ext.ptr(q), _ext.ptr(cache), _ext.ptr(block_table), ctypes.c_int(block_table.stride(0)),
                                  _ext.ptr(seqlens), _ext.ptr(sinks.float().contiguous() if sinks is not None else None),
                                  _ext.ptr(out), _ext.ptr(part_o), _ext.ptr(part_ml), ctypes.c_int(B), ctypes.c_int(Hq),
                                  ctypes.c_int(num_kv_heads), ctypes.c_int(D), ctypes.c_int(page), ctypes.c_int(window),
                                  ctypes.c_float(scale), ctypes.c_int(num_splits), _ext.stream())
    _ext.check(rc, "bg_gqa_decode", kernels=2 if num_splits > 1 else 1)
    return out


def mha_prefill_work(cu_seqlens: Sequence[int], ctx_lens: Sequence[int], k_starts: Sequence[int]) -> torch.Tensor:
    """Work list of the expanded-prefill kernel: one row (q_row0, n_q, k_row0, kv0) per 128-query tile; query i
    of a tile sees the first kv0 + i keys of its sequence, whose key rows start at ``k_starts[seq]``.  Longest
    key ranges first."""
    rows = []
    for i in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        for q0 in range(a, b, 128):
            rows.append((q0, min(128, b - q0), int(k_starts[i]), int(ctx_lens[i]) + (q0 - a) + 1))
    rows.sort(key=lambda r: -(r[3] + r[1]))
    return torch.tensor(rows, dtype=torch.int32).view(-1, 4)


def mha_prefill(q: torch.Tensor, kv: torch.Tensor, kpe: torch.Tensor, work: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal varlen attention in the expanded MLA form.  q [Tq, H, 192] (nope | roped pe); kv [Tk, H, 256]
    (key nope | value, the kv_b projection of the latent rows); kpe [Tk, >= 64] (roped shared key part in the
    first 64 columns, may be a strided view); ``work`` from ``mha_prefill_work`` -> [Tq, H, 128]."""
    Tq, H, _ = q.shape
    Tk = kv.shape[0]
    if not (q.is_cuda and q.dtype == torch.bfloat16):
        out = torch.zeros(Tq, H, 128, dtype=q.dtype)
        kf = torch.cat([kv[..., :128].float(), kpe[:, None, :64].float().expand(Tk, H, 64)], -1)
        vf = kv[..., 128:].float()
        for q0, nq, k0, kv0 in work.tolist():
            for i in range(nq):
                n = kv0 + i
                s = torch.einsum("hd,khd->hk", q[q0 + i].float(), kf[k0:k0 + n]) * scale
                out[q0 + i] = torch.einsum("hk,khd->hd", torch.softmax(s, -1), vf[k0:k0 + n]).to(q.dtype)
        return out
    assert q.is_contiguous() and kv.is_contiguous() and kpe.stride(1) == 1
    out = torch.empty(Tq, H, 128, dtype=torch.bfloat16, device=q.device)
    work = work.to(q.device)
    rc = _ext.lib().bg_mha_prefill(_ext.ptr(q), _ext.ptr(kv), _ext.ptr(kpe), ctypes.c_longlong(kpe.stride(0)), _ext.ptr(out),
                                   _ext.ptr(work), ctypes.c_int(work.shape[0]), ctypes.c_int(Tq), ctypes.c_int(Tk),
                                   ctypes.c_int(H), ctypes.c_float(scale), _ext.ptr(_ext.status_word(q.device)),
                                   _ext.stream())
    _ext.check(rc, "bg_mha_prefill")
    return out
