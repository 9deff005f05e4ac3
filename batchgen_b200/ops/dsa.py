"""DSA sparse-attention indexer operators (GPU path; the fp32 references live in ``ops.ref``).

``index_k_write``   fused LayerNorm + RoPE + e4m3 quantisation + paged store of the index keys
``indexer_select``  FP8 scores over the paged index keys on tcgen05, then exact top-k by radix select
``sparse_mla_decode`` gathers the selected latent rows into a dense buffer and runs the paged MLA kernel on it
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _ext

FP8 = torch.float8_e4m3fn


def supported(index_heads: int, index_dim: int, page: int) -> bool:
    return index_heads == 32 and index_dim == 128 and page == 64


def index_k_write(k, ln_w, ln_b, positions, cos_table, sin_table, rope: int, interleaved: bool, slot_mapping,
                  cache_k, cache_s, eps: float = 1e-6) -> None:
    """k [T, 128] bf16 (row stride allowed) -> cache_k [P, 64, 128] e4m3, cache_s [P, 64] fp32 at ``slot_mapping``."""
    T = k.shape[0]
    assert k.dtype == torch.bfloat16 and k.stride(1) == 1 and cache_k.is_contiguous() and cache_s.is_contiguous()
    rc = _ext.lib().bg_index_k_write(_ext.ptr(k), ctypes.c_int(k.stride(0)), _ext.ptr(ln_w), _ext.ptr(ln_b),
                                     _ext.ptr(positions), _ext.ptr(cos_table), _ext.ptr(sin_table), ctypes.c_int(rope),
                                     ctypes.c_int(int(interleaved)), _ext.ptr(slot_mapping), _ext.ptr(cache_k),
                                     _ext.ptr(cache_s), ctypes.c_int(T), ctypes.c_float(eps), _ext.stream())
    _ext.check(rc, "bg_index_k_write")


def quantize_index_q(q: torch.Tensor, gates: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B, 32, 128] -> (e4m3 q, gates with the per-head q scale folded in)."""
    amax = q.float().abs().amax(-1).clamp_min(1e-4)
    s = amax / 448.0
    q8 = (q.float() / s.unsqueeze(-1)).clamp(-448, 448).to(FP8)
    return q8.contiguous(), (gates.float() * s).contiguous()


def index_q_prepare(q: torch.Tensor, positions: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
                    rope: int, interleaved: bool, gates: torch.Tensor, gate_mul: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [T, 32, 128] bf16 (the index-query projection) -> (RoPE on the leading ``rope`` dims, e4m3 per head,
    ``gates * gate_mul`` with the per-head scale folded in): one kernel for rotate + quantise + gate scaling."""
    T, H, D = q.shape
    assert q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D and gates.dtype == torch.float32
    assert gates.is_contiguous() and positions.dtype == torch.int32
    q8 = torch.empty(T, H, D, dtype=FP8, device=q.device)
    g = torch.empty(T, H, dtype=torch.float32, device=q.device)
    rc = _ext.lib().bg_index_q_prepare(_ext.ptr(q), ctypes.c_longlong(q.stride(0)), _ext.ptr(positions),
                                       _ext.ptr(cos_table), _ext.ptr(sin_table), ctypes.c_int(rope),
                                       ctypes.c_int(int(interleaved)), _ext.ptr(gates), ctypes.c_float(gate_mul),
                                       _ext.ptr(q8), _ext.ptr(g), ctypes.c_int(T), ctypes.c_int(H), _ext.stream())
    _ext.check(rc, "bg_index_q_prepare")
    return q8, g


def indexer_scores(q8, gates, cache_k, cache_s, block_table, lengths, max_len: int) -> torch.Tensor:
    """-> fp32 scores [B, max_len] (entries past a row's length are undefined)."""
    B = q8.shape[0]
    P, S, D = cache_k.shape
    ld = (max_len + 3) // 4 * 4
    scores = torch.empty(B, ld, dtype=torch.float32, device=q8.device)
    rc = _ext.lib().bg_indexer_scores(_ext.ptr(q8), _ext.ptr(gates), _ext.ptr(cache_k), ctypes.c_longlong(P * S),
                                      _ext.ptr(cache_s), _ext.ptr(block_table), ctypes.c_int(block_table.stride(0)),
                                      _ext.ptr(lengths), _ext.ptr(scores), ctypes.c_longlong(ld), ctypes.c_int(B),
                                      ctypes.c_int(max_len), ctypes.c_int(_ext.num_sms(q8.device)),
                                      _ext.ptr(_ext.status_word(q8.device)), _ext.stream())
    _ext.check(rc, "bg_indexer_scores")
    return scores


def topk_select(scores: torch.Tensor, lengths: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact top-k positions per row (all positions when the row is no longer than k); order is arbitrary."""
    B = scores.shape[0]
    idx = torch.zeros(B, k, dtype=torch.int32, device=scores.device)
    n = torch.empty(B, dtype=torch.int32, device=scores.device)
    rc = _ext.lib().bg_topk_select(_ext.ptr(scores), ctypes.c_longlong(scores.stride(0)), _ext.ptr(lengths),
                                   ctypes.c_int(k), _ext.ptr(idx), ctypes.c_int(k), _ext.ptr(n), ctypes.c_int(B),
                                   _ext.stream())
    _ext.check(rc, "bg_topk_select")
    return idx, n


def indexer_select(q, gates, cache_k, cache_s, block_table, lengths, topk: int, max_len: int, prepared: bool = False):
    """``prepared``: ``q`` / ``gates`` already come from ``index_q_prepare`` (e4m3 queries, scaled gates)."""
    q8, g = (q, gates) if prepared else quantize_index_q(q, gates)
    scores = indexer_scores(q8, g, cache_k, cache_s, block_table, lengths, max_len)
    return topk_select(scores, lengths, topk)


def sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora):
    """MLA over selected positions: gather rows [B, K, 576] (K padded to whole pages) then the paged kernel."""
    from .mla_kernel import mla_decode_tc
    B = q_abs.shape[0]
    if B > 512:                                   # bound the dense gather buffer (prefill: one row per query)
        outs = [sparse_mla_decode(q_abs[i:i + 512], q_pe[i:i + 512], cache, block_table[i:i + 512], sel_idx[i:i + 512],
                                  sel_len[i:i + 512], scale, kv_lora) for i in range(0, B, 512)]
        return torch.cat(outs, 0)
    P, S, D = cache.shape
    K = (sel_idx.shape[1] + S - 1) // S * S
    dense = torch.empty(B, K, D, dtype=cache.dtype, device=cache.device)     # the gather zero-fills what is read
    rc = _ext.lib().bg_gather_rows(_ext.ptr(cache), _ext.ptr(block_table), ctypes.c_int(block_table.stride(0)),
                                   _ext.ptr(sel_idx), ctypes.c_int(sel_idx.stride(0)), _ext.ptr(sel_len),
                                   _ext.ptr(dense), ctypes.c_int(D * cache.element_size()), ctypes.c_int(S),
                                   ctypes.c_int(K), ctypes.c_int(B), _ext.stream())
    _ext.check(rc, "bg_gather_rows")
    pages = K // S
    bt = torch.arange(B * pages, dtype=torch.int32, device=cache.device).view(B, pages)
    return mla_decode_tc(q_abs, q_pe, dense.view(B * pages, S, D), bt, sel_len.to(torch.int32), scale, kv_lora)
