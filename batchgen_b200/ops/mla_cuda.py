"""CUDA entry points of the MLA attention operators.

``mla_decode`` / ``mla_prefill`` run the tcgen05 paged-latent kernel (``csrc/mla_tcgen05.cuh``, C entry points in
``csrc/mla_tcgen05.cu``).  Geometries the kernel does not cover (test-sized latent widths) have a batched library
path (gather + bmm) that is also the numerics cross-check used by the GPU tests; it runs only when
``ops.policy`` allows it and raises otherwise.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _ext
from .policy import library_fallback


def _why(q_abs, q_pe, cache, kv_lora) -> str:
    return (f"dtype {q_abs.dtype}, kv_lora {kv_lora}, rope {q_pe.shape[-1]}, page {cache.shape[1]}, "
            f"heads {q_abs.shape[1]}; the kernel needs bf16, 512 + 64, 64-token pages, heads % 8 == 0")


def _gather_padded(cache: torch.Tensor, block_table: torch.Tensor, max_len: int) -> torch.Tensor:
    P, S, D = cache.shape
    npg = (max_len + S - 1) // S
    pages = cache[block_table[:, :npg].long()]                 # [B, npg, S, D]
    return pages.reshape(block_table.shape[0], npg * S, D)[:, :max_len]


def mla_decode_lib(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora):
    """Library (bmm) implementation: the baseline the hand-written kernel is measured against."""
    B, H, _ = q_abs.shape
    Lmax = int(seqlens.max().item())
    kv = _gather_padded(cache, block_table, Lmax)
    c, kpe = kv[..., :kv_lora], kv[..., kv_lora:]
    s = (torch.bmm(q_abs, c.transpose(1, 2)).float() + torch.bmm(q_pe, kpe.transpose(1, 2)).float()) * scale
    mask = torch.arange(Lmax, device=q_abs.device).unsqueeze(0) >= seqlens.unsqueeze(1)
    s = s.masked_fill(mask.unsqueeze(1), float("-inf"))
    p = torch.softmax(s, dim=-1).to(q_abs.dtype)
    return torch.bmm(p, c)


def mla_decode(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora):
    if _kernel_supports(q_abs, q_pe, cache, kv_lora):
        from .mla_kernel import mla_decode_tc
        return mla_decode_tc(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora)
    library_fallback("mla_decode", _why(q_abs, q_pe, cache, kv_lora))
    return mla_decode_lib(q_abs, q_pe, cache, block_table, seqlens, scale, kv_lora)


def _kernel_supports(q_abs, q_pe, cache, kv_lora) -> bool:
    """The tcgen05 kernel covers the production geometry: bf16, 512 + 64 latent row, 64-token pages,
    a multiple of 8 heads per rank.  Other (test-sized) geometries use the library path."""
    return (q_abs.dtype == torch.bfloat16 and kv_lora == 512 and q_pe.shape[-1] == 64 and cache.shape[1] == 64
            and cache.dtype == torch.bfloat16 and q_abs.shape[1] % 8 == 0 and cache.is_contiguous())


def mla_prefill(q_abs, q_pe, cache, block_table, cu_seqlens: Sequence[int], ctx_lens: Sequence[int], scale, kv_lora):
    if _kernel_supports(q_abs, q_pe, cache, kv_lora):
        from .mla_kernel import mla_prefill_tc
        return mla_prefill_tc(q_abs, q_pe, cache, block_table, cu_seqlens, ctx_lens, scale, kv_lora)
    library_fallback("mla_prefill", _why(q_abs, q_pe, cache, kv_lora))
    return mla_prefill_lib(q_abs, q_pe, cache, block_table, cu_seqlens, ctx_lens, scale, kv_lora)


def mla_prefill_lib(q_abs, q_pe, cache, block_table, cu_seqlens: Sequence[int], ctx_lens: Sequence[int], scale,
                    kv_lora):
    """Varlen causal absorbed MLA.  Per sequence: one bmm over its cached rows with a causal mask
    (chunked over queries to bound the score matrix)."""
    T, H, _ = q_abs.shape
    out = torch.empty(T, H, kv_lora, dtype=q_abs.dtype, device=q_abs.device)
    P, S, D = cache.shape
    for i in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        n = b - a
        if n == 0:
            continue
        ctx = int(ctx_lens[i])
        L = ctx + n
        npg = (L + S - 1) // S
        kv = cache[block_table[i, :npg].long()].reshape(npg * S, D)[:L]
        c, kpe = kv[:, :kv_lora], kv[:, kv_lora:]
        chunk = max(1, min(n, (64 << 20) // max(1, H * L)))
        for q0 in range(0, n, chunk):
            q1 = min(n, q0 + chunk)
            qa = q_abs[a + q0: a + q1].transpose(0, 1)            # [H, m, 512]
            qp = q_pe[a + q0: a + q1].transpose(0, 1)
            s = (torch.matmul(qa, c.t()).float() + torch.matmul(qp, kpe.t()).float()) * scale
            qpos = torch.arange(q0, q1, device=s.device).unsqueeze(-1) + ctx
            kpos = torch.arange(L, device=s.device).unsqueeze(0)
            s = s.masked_fill((kpos > qpos).unsqueeze(0), float("-inf"))
            p = torch.softmax(s, dim=-1).to(q_abs.dtype)
            out[a + q0: a + q1] = torch.matmul(p, c).transpose(0, 1)
    return out


def sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora):
    if _kernel_supports(q_abs, q_pe, cache, kv_lora):
        from . import dsa
        return dsa.sparse_mla_decode(q_abs.contiguous(), q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora)
    library_fallback("sparse_mla_decode", _why(q_abs, q_pe, cache, kv_lora))
    return sparse_mla_decode_lib(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora)


def sparse_mla_decode_lib(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora):
    B, H, _ = q_abs.shape
    P, S, D = cache.shape
    K = sel_idx.shape[1]
    posn = sel_idx.long().clamp_min(0)
    slots = torch.gather(block_table.long(), 1, posn // S) * S + posn % S      # [B, K]
    kv = cache.view(P * S, D)[slots]                                           # [B, K, D]
    c, kpe = kv[..., :kv_lora], kv[..., kv_lora:]
    s = (torch.bmm(q_abs, c.transpose(1, 2)).float() + torch.bmm(q_pe, kpe.transpose(1, 2)).float()) * scale
    mask = torch.arange(K, device=q_abs.device).unsqueeze(0) >= sel_len.unsqueeze(1)
    s = s.masked_fill(mask.unsqueeze(1), float("-inf"))
    p = torch.softmax(s, dim=-1).to(q_abs.dtype)
    return torch.bmm(p, c)
