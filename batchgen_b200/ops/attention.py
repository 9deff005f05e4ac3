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
