"""MoE building blocks: router, local dispatch (permute + gather + quant), grouped expert GEMMs,
weighted combine.  ``experts_forward`` runs the expert stack of one rank over the tokens routed to
its local experts; it is shared by the single-GPU model, the NCCL all-gather/reduce-scatter
baseline and (for the post-dispatch part) the fused expert-parallel path.

Reference parity: the dataflow is gate -> dispatch -> act-quant -> grouped S1 (gate+up+SiLU) ->
quant -> grouped S3 (down) -> weighted reduce, as in batchgen/models/glm/glm5/model.py:2391-2508
and batchgen/moe/grouped_fp8_blockwise_moe.py.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _ext, fused, gemm, ref

FP8 = torch.float8_e4m3fn
ROW_ALIGN = 128  # grouped segments start on tile boundaries of the tcgen05 GEMM


@dataclass
class ExpertWeights:
    """Stacked weights of the experts one rank owns.

    quant == "none":      w13 [E, 2I, Kh], w2 [E, Hout, I] in the compute dtype.
    quant == "fp8_block": w13/w2 e4m3 with 128x128 scales w13_s [E, 2I/128, Kh/128], w2_s;
                          on CUDA, w13 rows are stored in the gate/up tile-interleaved order.
    quant == "mxfp4":     w13/w2 packed e2m1 (uint8, two values per byte) with e8m0 scales per 32
                          (w13 [E, 2I, Kh/2], w13_s [E, 2I, Kh/32]); same interleave rule on CUDA.
    quant == "int4":      w13/w2 packed offset-binary int4 with bf16 scales per 32 (same shapes).
    """
    w13: torch.Tensor
    w2: torch.Tensor
    w13_s: Optional[torch.Tensor] = None
    w2_s: Optional[torch.Tensor] = None
    quant: str = "none"
    interleaved: bool = False
    activation: str = "silu"             # silu | swiglu_clamped (GPT-OSS) | silu_limit (DeepSeek-V4: clamp, then SiLU(gate) * up)
    act_limit: float = 0.0               # clamp of silu_limit (0 = none)

    @property
    def num_experts(self) -> int:
        return self.w13.shape[0]

    def to_device_layout(self, force: bool = False) -> "ExpertWeights":
        """Reorder w13 rows for the fused SiLU epilogue (quantised experts; on CUDA tensors, or on host tensors
        that will be streamed to the GPU when ``force``)."""
        if self.quant not in ("fp8_block", "mxfp4", "int4") or self.interleaved or not (self.w13.is_cuda or force):
            return self
        perm = gemm.interleave_gate_up_rows(self.w13.shape[1], self.w13.device)
        if self.activation == "silu_limit" and self.act_limit > 0:
            return self                          # the clamp is not part of the fused epilogue: natural row order
        if self.quant in ("mxfp4", "int4"):
            if self.activation != "silu":
                return self                      # other activations run unfused: natural row order
            self.w13 = self.w13[:, perm].contiguous()
            self.w13_s = self.w13_s[:, perm].contiguous()
        else:
            self.w13 = self.w13.view(torch.uint8)[:, perm].contiguous().view(FP8)
        self.interleaved = True
        return self


def router_logits(hidden: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 router logits [T, E] = hidden @ weight^T (weight [E, H]).  On the GPU: the bf16 tcgen05 GEMM with
    an fp32 epilogue (the bf16 copy of the router weight is made once per weight tensor)."""
    if hidden.is_cuda and hidden.dtype == torch.bfloat16:
        # the bf16 copy rides on the weight tensor object itself (a cache keyed by address would serve a stale copy
        # once the allocator hands the address of a freed router weight to a new model)
        w = getattr(weight, "_bg_bf16", None)
        if w is None:
            w = weight if weight.dtype == torch.bfloat16 and weight.is_contiguous() else weight.to(torch.bfloat16).contiguous()
            weight._bg_bf16 = w
        if hidden.shape[1] % 64 == 0 and hidden.stride(1) == 1 and hidden.stride(0) == hidden.shape[1]:
            return gemm.bf16_gemm(hidden, w, fp32_out=True)
        from .policy import library_fallback
        library_fallback("router_logits", f"hidden {tuple(hidden.shape)} strides {hidden.stride()}; the GEMM needs "
                                          "contiguous rows with K % 64 == 0")
        return torch.mm(hidden, w.t(), out_dtype=torch.float32)
    return hidden.float() @ weight.float().t()


_SCORING_MODES = {"sigmoid": 0, "softmax": 1, "softmax_all": 2, "sqrtsoftplus": 3}


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int = 1,
                topk_group: int = 1, norm_topk_prob: bool = True, scale: float = 1.0, scoring: str = "sigmoid",
                num_valid: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (idx [T, k] int32, w [T, k] fp32).  ``num_valid`` (device int32 scalar) marks rows >= it as
    padding: they get idx -1 / weight 0 and are ignored by dispatch."""
    if not logits.is_cuda:
        idx, w = ref.router_topk(logits, bias, top_k, n_group, topk_group, norm_topk_prob, scale, scoring)
        if num_valid is not None:
            nv = int(num_valid)
            idx[nv:] = -1
            w[nv:] = 0
        return idx, w
    T, E = logits.shape
    logits = logits.contiguous()
    idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    rc = _ext.lib().bg_router_topk(_ext.ptr(logits), _ext.ptr(bias), _ext.ptr(idx), _ext.ptr(w), ctypes.c_int(T),
                                   ctypes.c_int(E), ctypes.c_int(top_k), ctypes.c_int(n_group),
                                   ctypes.c_int(topk_group), ctypes.c_int(int(norm_topk_prob)), ctypes.c_float(scale),
                                   ctypes.c_int(_SCORING_MODES[scoring]), _ext.ptr(num_valid), _ext.stream())
    _ext.check(rc, "bg_router_topk")
    return idx, w


def permute(topk_idx: torch.Tensor, lo: int, hi: int, num_valid: Optional[torch.Tensor] = None,
            align: int = ROW_ALIGN):
    """Group (token, k) pairs by local expert.  -> (src_row [cap] int32, pos [T, k] int32,
    offsets [El+1] int32).  Rows past offsets[El] are unused capacity.  ``align``: segment starts are multiples of
    it (128 = the row tile of the wide GEMM kernels; 32 = the token tile of the swapped-operand kernel, which keeps
    the padded capacity, and with it the per-row kernels' grids, small at decode sizes)."""
    T, K = topk_idx.shape
    El = hi - lo
    if not topk_idx.is_cuda:
        idx = topk_idx
        if num_valid is not None:
            idx = idx.clone()
            idx[int(num_valid):] = -1
        src, pos, off = ref.moe_permute(idx, hi, lo, hi, align=1)
        return src.to(torch.int32), pos.to(torch.int32), off.to(torch.int32)
    cap = (T * K + align - 1) // align * align + El * align
    dev = topk_idx.device
    offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
    cursor = torch.empty(El, dtype=torch.int32, device=dev)
    pos = torch.empty(T, K, dtype=torch.int32, device=dev)
    src = torch.empty(cap, dtype=torch.int32, device=dev)
    rc = _ext.lib().bg_moe_permute(_ext.ptr(topk_idx), ctypes.c_int(T), ctypes.c_int(K), ctypes.c_int(lo),
                                   ctypes.c_int(hi), ctypes.c_int(align), _ext.ptr(offsets), _ext.ptr(cursor),
                                   _ext.ptr(pos), _ext.ptr(src), ctypes.c_int(cap), _ext.ptr(num_valid), _ext.stream())
    _ext.check(rc, "bg_moe_permute", kernels=2)
    offsets.real_counts = cursor          # after the scatter pass: rows really present in each segment
    return src, pos, offsets


def gather_quant(hidden: torch.Tensor, src_row: torch.Tensor, offsets: torch.Tensor, pow2_scale: bool = False,
                 zero_padding: bool = True):
    """Gather hidden rows into expert-grouped order and quantise -> (q [cap, K] e4m3, s [cap, K/128]).
    Padding rows of a segment become zeros, or stay undefined with ``zero_padding=False`` (for a grouped
    GEMM that is given the real row counts)."""
    K = hidden.shape[1]
    if not hidden.is_cuda:
        rows = hidden[src_row.clamp_min(0).long()].float()
        rows = torch.where((src_row >= 0).unsqueeze(-1), rows, torch.zeros_like(rows))
        return ref.act_quant(rows, 128, pow2_scale)
    cap = src_row.shape[0]
    q = torch.empty(cap, K, dtype=FP8, device=hidden.device)
    s = fused._scale_buffer(cap, K // 128, hidden.device)
    rc = _ext.lib().bg_moe_gather_quant(_ext.ptr(hidden), ctypes.c_int(hidden.stride(0)), _ext.ptr(src_row),
                                        _ext.ptr(offsets[-1:]), _ext.ptr(q), _ext.ptr(s), ctypes.c_int(s.stride(1)),
                                        ctypes.c_int(cap), ctypes.c_int(K), ctypes.c_int(int(pow2_scale)),
                                        ctypes.c_int(int(zero_padding)), _ext.stream())
    _ext.check(rc, "bg_moe_gather_quant")
    return q, s


def combine(y: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor, extra: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out[t] = (extra[t]) + sum_k weights[t, k] * y[pos[t, k]] in ascending k."""
    if not y.is_cuda:
        out = ref.moe_combine(y, pos.long(), weights, torch.float32)
        if extra is not None:
            out = out + extra.float()
        return out.to(out_dtype or y.dtype)
    T, K = pos.shape
    H = y.shape[1]
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty(T, H, dtype=out_dtype, device=y.device)
    rc = _ext.lib().bg_moe_combine(_ext.ptr(y), ctypes.c_int(y.stride(0)), _ext.ptr(pos), _ext.ptr(weights),
                                   _ext.ptr(extra), ctypes.c_int(extra.stride(0) if extra is not None else 0),
                                   _ext.ptr(out), ctypes.c_int(out.stride(0)), ctypes.c_int(T), ctypes.c_int(K),
                                   ctypes.c_int(H), ctypes.c_int(1 if out_dtype == torch.float32 else 0),
                                   _ext.stream())
    _ext.check(rc, "bg_moe_combine")
    return out


def _activation(gate_up: torch.Tensor, kind: str, limit: float = 0.0) -> torch.Tensor:
    if kind == "swiglu_clamped":
        return ref.swiglu_clamped(gate_up)
    if kind == "silu_limit" and limit > 0:
        I = gate_up.shape[-1] // 2
        g, u = gate_up[..., :I].float().clamp(max=limit), gate_up[..., I:].float().clamp(-limit, limit)
        return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)
    return ref.silu_mul(gate_up)


def grouped_experts(xq, xs, offsets: torch.Tensor, ew: ExpertWeights, x_dense: Optional[torch.Tensor] = None,
                    timer=None, counts: Optional[torch.Tensor] = None, row_src: Optional[torch.Tensor] = None,
                    rows_hint: Optional[int] = None):
    """Run gate/up -> activation -> down for rows already grouped by expert.  fp8 path takes
    (xq, xs); the unquantised path takes ``x_dense``.  Returns y [rows, Hout].  With ``counts`` (real rows
    per segment) and ``row_src`` (negative on padding rows) the padding rows are skipped end to end."""
    if timer is None:
        from ..utils.timing import null_timer
        timer = null_timer()
    if ew.quant == "fp8_block":
        if xq.is_cuda:
            assert ew.interleaved, "call ExpertWeights.to_device_layout() after loading"
            with timer.timed("moe.s1_gemm"):
                act = gemm.grouped_fp8_gemm(xq, xs, ew.w13, ew.w13_s, offsets, silu_mul=True, counts=counts,
                                            rows_hint=rows_hint)
            with timer.timed("moe.act_quant"):
                aq, as_ = fused.act_quant(act, valid_rows=offsets[-1:], row_src=row_src)
            with timer.timed("moe.s3_gemm"):
                return gemm.grouped_fp8_gemm(aq, as_, ew.w2, ew.w2_s, offsets, counts=counts, rows_hint=rows_hint)
        gu = ref.grouped_fp8_gemm(xq, xs, ew.w13, ew.w13_s, offsets)
        act = _activation(gu, ew.activation, ew.act_limit)
        aq, as_ = ref.act_quant(act)
        return ref.grouped_fp8_gemm(aq, as_, ew.w2, ew.w2_s, offsets)
    if ew.quant in ("mxfp4", "int4"):
        # W4A16, groups of 32: one tcgen05 kernel, two expansions (e2m1 x e8m0 scale, or offset-binary int4 x bf16 scale)
        if ew.quant == "mxfp4":
            from .mxfp4 import grouped_mxfp4_gemm as grouped_w4
        else:
            from .int4 import grouped_int4_gemm as grouped_w4
        x = x_dense
        if x.is_cuda and ew.interleaved:
            with timer.timed("moe.s1_gemm"):
                act = grouped_w4(x, ew.w13, ew.w13_s, offsets, silu_mul=True)
        else:
            with timer.timed("moe.s1_gemm"):
                gu = grouped_w4(x, ew.w13, ew.w13_s, offsets)
            act = _activation(gu, ew.activation, ew.act_limit).to(x.dtype)
        with timer.timed("moe.s3_gemm"):
            return grouped_w4(act, ew.w2, ew.w2_s, offsets)
    # unquantised experts (CPU fp32 oracle path and bf16 debugging)
    x = x_dense
    out = torch.zeros(x.shape[0], ew.w2.shape[1], dtype=x.dtype, device=x.device)
    off = offsets.tolist()
    for e in range(ew.num_experts):
        a, b = off[e], off[e + 1]
        if b > a:
            gu = x[a:b] @ ew.w13[e].t()
            out[a:b] = _activation(gu, ew.activation, ew.act_limit) @ ew.w2[e].t()
    return out


def experts_forward(hidden: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, ew: ExpertWeights,
                    expert_lo: int, expert_hi: int, extra: Optional[torch.Tensor] = None,
                    num_valid: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                    timer=None, before_combine=None) -> torch.Tensor:
    """Partial MoE output of one rank: sum over the (token, k) pairs whose expert is local (+ ``extra``).
    ``before_combine`` is called right before the combine reads ``extra`` (it may come from another stream)."""
    if timer is None:
        from ..utils.timing import null_timer
        timer = null_timer()
    align = ROW_ALIGN
    if ew.quant == "fp8_block" and hidden.is_cuda and ew.interleaved:
        # decode-sized steps run on the swapped-operand kernel (32-token tiles): 32-row segment alignment keeps the
        # padded capacity close to the real row count
        pairs = topk_idx.shape[0] * topk_idx.shape[1]
        if gemm.use_swapab(pairs / max(expert_hi - expert_lo, 1), ew.w13.shape[1], ew.w13.shape[2]):
            align = 32
    with timer.timed("moe.permute"):
        src, pos, offsets = permute(topk_idx, expert_lo, expert_hi, num_valid, align=align)
    if ew.quant == "fp8_block":
        counts = getattr(offsets, "real_counts", None)
        with timer.timed("moe.gather_quant"):
            xq, xs = gather_quant(hidden, src, offsets, zero_padding=counts is None)
        y = grouped_experts(xq, xs, offsets, ew, timer=timer, counts=counts,
                            row_src=src if counts is not None else None,
                            rows_hint=(hidden.shape[0] * topk_idx.shape[1] if counts is not None else None))
    else:
        rows = hidden[src.clamp_min(0).long()]
        rows = torch.where((src >= 0).unsqueeze(-1), rows, torch.zeros_like(rows))
        y = grouped_experts(None, None, offsets, ew, x_dense=rows)
    with timer.timed("moe.combine"):
        if before_combine is not None:
            before_combine()
        return combine(y, pos, topk_w, extra, out_dtype or hidden.dtype)
