"""GEMM entry points: block-scaled FP8 and bf16, dense and grouped.

CUDA tensors go to the tcgen05 kernel (``csrc/gemm_tcgen05.cu``); CPU tensors go to the fp32
reference.  Activation scales are consumed in *row-contiguous-per-block* layout
(``scale[kb, m]``), which is what the fused quantisation kernels emit; a ``[T, KB]`` contiguous
tensor is transposed on the fly.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _ext, ref

KIND_FP8, KIND_BF16 = 0, 1
EPI_STORE, EPI_SILU_MUL, EPI_STORE_F32 = 0, 1, 2


def interleave_gate_up_rows(n_rows: int, device=None) -> torch.Tensor:
    """Row permutation that turns a [2I, K] gate-then-up weight into the tile-interleaved layout
    the fused SiLU epilogue reads: every 64 consecutive rows hold 32 gate rows followed by the 32
    up rows of the same output columns."""
    I = n_rows // 2
    assert I % 128 == 0, "intermediate size must be a multiple of 128"
    j = torch.arange(I, device=device)
    blk, within = j // 32, j % 32
    idx = torch.empty(n_rows, dtype=torch.long, device=device)
    idx[blk * 64 + within] = j
    idx[blk * 64 + 32 + within] = I + j
    return idx


def _scales_kb_major(xs: torch.Tensor):
    """Return (tensor, stride) with scale(m, kb) at data[kb * stride + m]."""
    if xs.dim() != 2:
        raise ValueError("activation scales must be 2-D [T, KB]")
    if xs.stride(0) == 1 or xs.shape[0] == 1:
        return xs, (xs.stride(1) if xs.shape[1] > 1 else xs.shape[0])
    t = xs.t().contiguous()  # [KB, T]
    return t, t.stride(0)


_WIDE = os.environ.get("BG_GEMM_WIDE", "auto")       # "0": always 128x128 tiles, "1": 128x256 whenever allowed
_SWAPAB = os.environ.get("BG_GEMM_SWAPAB", "auto")   # "0": never, "1": whenever allowed; auto: few rows per weight matrix
SWAPAB_MAX_ROWS = 32                                 # rows per weight matrix (on average) up to which weights go on the M side


def use_swapab(rows_per_matrix: float, N: int, K: int) -> bool:
    """The swapped-operand kernel (weights on the MMA M side, 32-token tiles) is the weight-streaming kernel of
    decode-sized steps: it wins while a weight matrix sees about one token tile."""
    if _SWAPAB == "0" or N % 128 or K % 128 or K // 128 > 160:
        return False
    return _SWAPAB == "1" or rows_per_matrix <= SWAPAB_MAX_ROWS


_hooks_pending = False     # set by the fused-communication layer right before a GEMM that consumes collective hooks


def hooks_pending() -> None:
    global _hooks_pending
    _hooks_pending = True


def _use_wide(kind, D, M, N, wide) -> bool:
    """128 x 256 tiles pay off when there are plenty of tiles to fill the SMs; GEMMs that consume collective
    hooks (rows stored to peers, flag waits) and bf16 operands stay on the 128 x 128 kernel."""
    global _hooks_pending
    if _hooks_pending:
        _hooks_pending = False
        return False
    if kind != KIND_FP8 or wide is False or _WIDE == "0" or not isinstance(D, torch.Tensor):
        return False
    if wide is True or _WIDE == "1":
        return True
    tiles = -(-M // 128) * -(-N // 128)
    return tiles >= 2 * _ext.num_sms(D.device)


def wide_enabled() -> bool:
    return _WIDE != "0"


_SPLITK = os.environ.get("BG_GEMM_SPLITK", "1")
_splitk_ws: dict = {}


def _ensure_splitk_workspace(device) -> None:
    """Dense GEMMs whose output has too few 128 x 128 tiles to fill the SMs (decode-sized projections, router
    logits) split K over several CTAs; their partial tiles and per-tile counters live in one scratch per device,
    handed to the launcher once (it may not allocate: the launch can be part of a stream capture)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key in _splitk_ws or _SPLITK == "0":
        return
    sms = _ext.num_sms(device)
    ws = torch.empty(4 * sms * 128 * 128, dtype=torch.float32, device=device)      # 4 x SMs partial tiles (38 MB)
    cnt = torch.zeros(4096, dtype=torch.int32, device=device)
    _splitk_ws[key] = (ws, cnt)
    L = _ext.lib()
    L.bg_gemm_set_splitk_ws.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int]
    with torch.cuda.device(device):
        rc = L.bg_gemm_set_splitk_ws(ctypes.c_void_p(ws.data_ptr()), ctypes.c_longlong(4 * sms),
                                     ctypes.c_void_p(cnt.data_ptr()), ctypes.c_int(cnt.numel()))
    _ext.check(rc, "bg_gemm_set_splitk_ws")


def _launch(kind, epi, A, sA, sa_stride, B, sB, D, offsets, groups, M, N, K, wide=None, counts=None, a_ready=None,
            swapab=False):
    """``a_ready`` = (flag pointer, epoch, epoch-base pointer, world): the rows of A are pushed by peers and the
    128 x 256 kernel's producer waits for every rank's arrival flag (only that kernel and the swapped-operand kernel
    take it this way)."""
    L = _ext.lib()
    if swapab and kind == KIND_FP8 and epi != EPI_STORE_F32:
        global _hooks_pending
        assert not _hooks_pending, "collective hooks belong to the 128 x 128 kernel"
        flag, epoch, base, world = a_ready if a_ready is not None else (ctypes.c_void_p(0), 0, ctypes.c_void_p(0), 1)
        rc = L.bg_gemm_fp8_swapab(ctypes.c_int(epi), _ext.ptr(A), _ext.ptr(sA), ctypes.c_int(sa_stride), _ext.ptr(B),
                                  _ext.ptr(sB), _ext.ptr(D), ctypes.c_int(D.stride(0)), _ext.ptr(offsets), _ext.ptr(counts),
                                  ctypes.c_int(groups), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                  ctypes.c_int(_ext.num_sms(A.device)), flag, ctypes.c_uint32(epoch),
                                  base, ctypes.c_int(world), _ext.ptr(_ext.status_word(A.device)), _ext.stream())
        _ext.check(rc, "bg_gemm_fp8_swapab")
        return
    if a_ready is not None or _use_wide(kind, D, M, N, wide):
        flag, epoch, base, world = a_ready if a_ready is not None else (ctypes.c_void_p(0), 0, ctypes.c_void_p(0), 1)
        rc = L.bg_gemm_fp8_n256(ctypes.c_int(epi), _ext.ptr(A), _ext.ptr(sA), ctypes.c_int(sa_stride), _ext.ptr(B),
                                _ext.ptr(sB), _ext.ptr(D), ctypes.c_int(D.stride(0)), _ext.ptr(offsets), _ext.ptr(counts),
                                ctypes.c_int(groups), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                ctypes.c_int(_ext.num_sms(A.device)), flag, ctypes.c_uint32(epoch),
                                base, ctypes.c_int(world), _ext.ptr(_ext.status_word(A.device)), _ext.stream())
        _ext.check(rc, "bg_gemm_fp8_n256")
        return
    if counts is not None:
        L.bg_gemm_set_counts(_ext.ptr(counts))
    _ensure_splitk_workspace(A.device)
    rc = L.bg_gemm(ctypes.c_int(kind), ctypes.c_int(epi), _ext.ptr(A), _ext.ptr(sA), ctypes.c_int(sa_stride),
                   _ext.ptr(B), _ext.ptr(sB), _ext.ptr(D), ctypes.c_int(D.stride(0)), _ext.ptr(offsets),
                   ctypes.c_int(groups), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                   ctypes.c_int(_ext.num_sms(A.device)), _ext.ptr(_ext.status_word(A.device)), _ext.stream())
    _ext.check(rc, "bg_gemm")


def fp8_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
             out: Optional[torch.Tensor] = None, silu_mul: bool = False, wide: Optional[bool] = None,
             swapab: Optional[bool] = None) -> torch.Tensor:
    """[T, K] e4m3 x [N, K] e4m3 -> [T, N] (bf16 on GPU).  With ``silu_mul`` the weight must be in
    the interleaved gate/up layout and the result has N/2 columns."""
    T, K = xq.shape
    N = wq.shape[0]
    if not xq.is_cuda:
        y = ref.fp8_gemm(xq, xs, wq, ws)
        if silu_mul:
            inv = torch.argsort(interleave_gate_up_rows(N))
            y = ref.silu_mul(y[:, inv])
        return y
    n_out = N // 2 if silu_mul else N
    if out is None:
        out = torch.empty(T, n_out, dtype=torch.bfloat16, device=xq.device)
    if T == 0:
        return out
    s, stride = _scales_kb_major(xs)
    if swapab is None:
        swapab = (not _hooks_pending) and wide is None and use_swapab(T / 2, N, K)     # up to two 32-token tiles
    _launch(KIND_FP8, EPI_SILU_MUL if silu_mul else EPI_STORE, xq, s, stride, wq, ws, out, None, 1, T, N, K, wide=wide,
            swapab=swapab)
    return out


def grouped_fp8_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
                     offsets: torch.Tensor, out: Optional[torch.Tensor] = None,
                     silu_mul: bool = False, counts: Optional[torch.Tensor] = None,
                     wide: Optional[bool] = None, a_ready=None, rows_hint: Optional[int] = None) -> torch.Tensor:
    """Ragged grouped GEMM.  xq: [R, K] rows grouped by expert, segment e = offsets[e]:offsets[e+1]
    (int32 on device, every start a multiple of 128 on the GPU path); wq: [E, N, K].  ``counts`` (int32 [E],
    device) gives the rows really present in each segment: padding rows are then neither stored nor, as
    whole tiles, computed (their output rows stay undefined).  ``rows_hint``: rows the caller expects to be really
    present in total (the padded row count R says little); few rows per expert select the swapped-operand kernel."""
    E, N, K = wq.shape
    R = xq.shape[0]
    if not xq.is_cuda:
        y = ref.grouped_fp8_gemm(xq, xs, wq, ws, offsets)
        if silu_mul:
            inv = torch.argsort(interleave_gate_up_rows(N))
            y = ref.silu_mul(y[:, inv])
        return y
    n_out = N // 2 if silu_mul else N
    if out is None:
        out = torch.empty(R, n_out, dtype=torch.bfloat16, device=xq.device)
    if R == 0:
        return out
    s, stride = _scales_kb_major(xs)
    assert offsets.dtype == torch.int32 and offsets.is_cuda
    if counts is not None:
        assert counts.dtype == torch.int32 and counts.is_cuda and counts.numel() >= E
    swapab = (not _hooks_pending) and wide is None and rows_hint is not None and use_swapab(rows_hint / max(E, 1), N, K)
    _launch(KIND_FP8, EPI_SILU_MUL if silu_mul else EPI_STORE, xq, s, stride, wq.view(E * N, K), ws, out,
            offsets, E, R, N, K, wide=wide, counts=counts, a_ready=a_ready, swapab=swapab)
    return out


def bf16_gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, fp32_out: bool = False) -> torch.Tensor:
    """[T, K] bf16 x [N, K] bf16 -> [T, N] bf16, or fp32 with ``fp32_out`` (fp32 accumulate in TMEM).  For a given
    shape the summation order is fixed (repeatable bit for bit); shapes with few output tiles split K over CTAs, so
    the order can differ between batch sizes."""
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        return y if fp32_out else y.to(x.dtype)
    T, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if fp32_out else torch.bfloat16, device=x.device)
    if T == 0:
        return out
    _launch(KIND_BF16, EPI_STORE_F32 if fp32_out else EPI_STORE, x, None, 0, w, None, out, None, 1, T, N, K)
    return out
