"""The decoder-only transformer shared by every supported family.

One class covers MLA (DeepSeek-V3/R1, GLM-5.x, Kimi) and GQA (GPT-OSS, MiniMax) attention, dense and
MoE feed-forward (sigmoid group-limited or softmax routing, shared expert, Kimi LatentMoE) and the
DSA sparse-attention indexer.  It is a pure function of (weights, KV cache, attention metadata):
all state lives in the caller's ``PagedKVCache``.

Tokens of a step are always flattened to ``[T]``; ``AttnMeta`` says how they map to sequences:

* prefill: ``cu_seqlens`` delimits each sequence's new tokens, ``ctx_lens`` counts tokens already
  cached before them (prefix hit / chunked prefill), ``slot_mapping`` says where each new token's KV
  row goes, ``block_table`` row i is sequence i's pages.
* decode: one token per sequence; ``seqlens`` includes the new token.

Parallelism is injected through ``comm`` (see ``parallel.comm``): attention heads, dense MLP and the
shared expert are tensor-parallel over ``tp`` ranks (partial sums reduced by ``comm.tp_reduce``), routed
experts are expert-parallel (``comm.moe``).  With ``comm is None`` everything is local.

Reference parity: batchgen/models/deepseek/deepseekv3/modeling_deepseek_v3.py (MLA + MoE layer
structure, gate :746-850), batchgen/models/glm/glm5/model.py:610-700 (DSA indexer oracle) and
:2391-2508 (decode MoE dataflow), batchgen/attention/mla/torch_backend.py (absorbed MLA math).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..config import ModelConfig
from ..ops import attention as attn_ops
from ..ops import fused, gemm, ref
from ..ops import kda as kda_ops
from ..ops import moe as moe_ops
from ..utils.timing import null_timer
from .weights import LayerWeights, Linear, ModelWeights, ParallelLayout


@dataclass
class AttnMeta:
    mode: str                                   # "prefill" | "decode"
    positions: torch.Tensor                     # [T] int32
    slot_mapping: torch.Tensor                  # [T] int64 flat KV slot of each new token (-1 = skip)
    block_table: torch.Tensor                   # [nseq, max_pages] int32
    seqlens: Optional[torch.Tensor] = None      # decode: [B] int32 lengths including the new token
    cu_seqlens: Optional[List[int]] = None      # prefill: [nseq + 1]
    ctx_lens: Optional[List[int]] = None        # prefill: tokens cached before this step
    logit_rows: Optional[torch.Tensor] = None   # rows of T whose logits are wanted (prefill: last tokens)
    num_valid: Optional[torch.Tensor] = None    # decode under CUDA graphs: device count of real rows
    dsa_selection: dict = field(default_factory=dict)  # layer -> (sel_idx, sel_len) reused by shared layers
    state_slots: Optional[torch.Tensor] = None  # KDA layers: [nseq] int32 state slot of each sequence (< 0 = skip)
    state_has_initial: Optional[torch.Tensor] = None  # prefill: [nseq] int32, 0 = start from a zero state
    _own_slots: Optional[torch.Tensor] = None   # slot mapping masked to this rank's rows (request-parallel decode)


class RopeTables:
    def __init__(self, cfg: ModelConfig, max_pos: int, device):
        d = cfg.qk_rope_head_dim if cfg.is_mla else cfg.head_dim
        inv = ref.rope_inv_freq(d, cfg.rope_theta, cfg.rope_scaling_factor, cfg.rope_original_max_pos,
                                cfg.rope_beta_fast, cfg.rope_beta_slow)
        pos = torch.arange(max_pos, dtype=torch.float32)
        ang = pos.unsqueeze(-1) * inv
        self.cos = ang.cos().to(device).contiguous()
        self.sin = ang.sin().to(device).contiguous()
        self.max_pos = max_pos


def linear(x, lin: Linear, xq=None, xs=None, silu_mul: bool = False):
    """y = x @ W^T.  FP8 weights consume the quantised activation (computed here unless passed in)."""
    if lin.is_fp8:
        if xq is None:
            xq, xs = fused.act_quant(x)
        if xq.is_cuda:
            return gemm.fp8_gemm(xq, xs, lin.w, lin.s, silu_mul=silu_mul and lin.interleaved)
        y = ref.fp8_gemm(xq, xs, lin.w, lin.s).to(x.dtype if x is not None else torch.float32)
        return y
    if x.is_cuda and x.dtype == torch.bfloat16 and lin.w.shape[1] % 64 == 0:
        return gemm.bf16_gemm(x.contiguous(), lin.w)
    if x.is_cuda:
        from ..ops.policy import library_fallback
        library_fallback("linear", f"x {tuple(x.shape)} {x.dtype}, K {lin.w.shape[1]}; the bf16 GEMM needs K % 64 == 0")
    return x @ lin.w.t()


class Transformer:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, layout: Optional[ParallelLayout] = None,
                 comm=None, max_positions: int = 8192):
        self.cfg = cfg
        self.w = weights
        self.layout = layout or ParallelLayout()
        self.comm = comm
        self.device = weights.embed.device
        self.dtype = weights.embed.dtype
        self.rope = RopeTables(cfg, max_positions, self.device)
        self.timer = null_timer()     # utils.timing.TimingStats when profiling
        # decode attention core split by request inside the TP group (static row ownership: row i belongs to rank
        # i // (T / world) for as long as it decodes); off by default because the engine may re-order rows
        self.attn_request_parallel = False
        self.streamer = None          # models.streaming.StreamedExperts when the routed experts live in host memory
        self.overlap_shared_expert = os.environ.get("BG_OVERLAP_SHARED", "1") != "0"   # decode: shared expert on a side stream
        self.expanded_prefill_min_tokens = 256   # below this the absorbed kernel is as fast and saves the kv_b GEMM

    # ------------------------------------------------------------------ helpers
    def _mlp(self, x, xq, xs, w13: Linear, w2: Linear):
        if w13.is_fp8 and x.is_cuda and w13.interleaved:
            act = linear(x, w13, xq, xs, silu_mul=True)
        else:
            gu = linear(x, w13, xq, xs)
            act = ref.swiglu_clamped(gu) if self.cfg.activation == "swiglu_clamped" else ref.silu_mul(gu)
        return linear(act, w2)

    def _norm(self, x, w, residual, quant):
        return fused.rmsnorm(x, w, self.cfg.rms_eps, residual=residual, quant=quant)

    def _lm_head(self, x) -> torch.Tensor:
        """fp32 logits = x @ lm_head^T: the bf16 tcgen05 GEMM with an fp32 epilogue on the GPU."""
        w = self.w.lm_head
        if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 64 == 0:
            return gemm.bf16_gemm(x.contiguous(), w, fp32_out=True)
        if x.is_cuda:
            from ..ops.policy import library_fallback
            library_fallback("lm_head", f"x {x.dtype}, weight {tuple(w.shape)} {w.dtype}")
        return (x @ w.t()).float()

    # ------------------------------------------------------------------ attention
    def _mla(self, l: int, lw: LayerWeights, x, xq, xs, meta: AttnMeta, cache) -> torch.Tensor:
        cfg = self.cfg
        T = x.shape[0]
        Hh = lw.w_uk.shape[0]
        tm = self.timer
        with tm.timed("attn.qkv_a_gemm", l):
            qkv_a = linear(x, lw.wqkv_a, xq, xs)
        o = self._mla_from_qkv_a(l, lw, qkv_a, x, meta, cache)
        with tm.timed("attn.o_proj", l):
            return linear(o, lw.wo)

    def _mla_from_qkv_a(self, l: int, lw: LayerWeights, qkv_a, x, meta: AttnMeta, cache) -> torch.Tensor:
        """Everything between the q_a/kv_a projection and o_proj: KV write, q path, attention over the
        paged latent cache, out-absorb.  Returns [T, local_heads * v_head_dim]."""
        cfg = self.cfg
        T = qkv_a.shape[0]
        tm = self.timer
        q_a, kv_a = qkv_a[:, : cfg.q_lora_rank], qkv_a[:, cfg.q_lora_rank:]
        with tm.timed("attn.kv_write_qnorm_qb_rope", l):
            self._mla_q(lw, q_a, kv_a, meta, cache, l)
        q, qn = self._q, self._qn
        if (meta.mode == "prefill" and lw.w_kvb is not None and q.is_cuda and T >= self.expanded_prefill_min_tokens
                and not any(meta.ctx_lens)):
            # long fresh prompts: attention over up-projected keys / values (3.4x fewer FLOPs than the
            # absorbed form); the latent rows were just written to the cache, read them back by slot
            with tm.timed("attn.core_prefill", l):
                lat = cache.latent(l).view(-1, cfg.kv_cache_dim)[meta.slot_mapping.clamp_min(0)]
                kvb = gemm.bf16_gemm(lat[:, : cfg.kv_lora_rank].contiguous(), lw.w_kvb)
                Hh = q.shape[1]
                key = (tuple(meta.cu_seqlens), T)
                if getattr(meta, "_mha_work_key", None) != key:
                    meta._mha_work = attn_ops.mha_prefill_work(meta.cu_seqlens, meta.ctx_lens, meta.cu_seqlens[:-1]).to(q.device)
                    meta._mha_work_key = key
                o = attn_ops.mha_prefill(q, kvb.view(T, Hh, 256), lat[:, cfg.kv_lora_rank:], meta._mha_work,
                                         cfg.softmax_scale)
                if meta.cu_seqlens[-1] < T:
                    o[meta.cu_seqlens[-1]:].zero_()      # padding rows of a sequence-parallel step belong to no sequence
            return o.reshape(T, -1)
        q_nope, q_pe = q[..., : cfg.qk_nope_head_dim], q[..., cfg.qk_nope_head_dim:]
        # absorb W_UK: [T, Hh, nope] x [Hh, nope, kv_lora] -> [T, Hh, kv_lora]
        rp = self._request_parallel(meta, T)
        with tm.timed("attn.q_absorb", l):
            if rp:      # both query parts in one [T, Hh, kv_lora + rope] buffer: the exchange moves it as it is
                qbuf = torch.empty(T, q.shape[1], cfg.kv_lora_rank + cfg.qk_rope_head_dim, dtype=q.dtype, device=q.device)
                q_abs = attn_ops.mla_q_absorb(q, lw.w_uk_t, cfg.qk_nope_head_dim, out=qbuf[..., : cfg.kv_lora_rank])
                qbuf[..., cfg.kv_lora_rank:] = q_pe
            else:
                q_abs = attn_ops.mla_q_absorb(q, lw.w_uk_t, cfg.qk_nope_head_dim)
        sel = None
        if cfg.has_dsa:
            with tm.timed("attn.dsa_indexer", l):
                sel = self._dsa_select(l, lw, x, qn, meta, cache)
        with tm.timed("attn.core_" + meta.mode, l):
            if rp:
                o_lat = self._mla_core_request_parallel(l, qbuf, meta, cache)
            else:
                o_lat = self._mla_core(l, lw, q_abs, q_pe, sel, meta, cache)
        # out-absorb W_UV: [T, Hh, kv_lora] x [Hh, v, kv_lora]^T -> [T, Hh * v]
        with tm.timed("attn.out_absorb", l):
            return attn_ops.mla_out_absorb(o_lat, lw.w_uv)

    def _mla_q(self, lw, q_a, kv_a, meta, cache, l):
        cfg = self.cfg
        T = q_a.shape[0]
        Hh = lw.w_uk.shape[0]
        slots = meta.slot_mapping
        if self._request_parallel(meta, T):
            # request-parallel attention core: a row's latent KV lives only on the rank that owns the row
            if meta._own_slots is None:
                W, r = self.layout.tp_size, self.layout.tp_rank
                own = torch.zeros(T, dtype=torch.bool, device=slots.device)
                own[r * (T // W):(r + 1) * (T // W)] = True
                meta._own_slots = torch.where(own, slots, torch.full_like(slots, -1))
            slots = meta._own_slots
        fused.mla_kv_write(kv_a, lw.kv_norm, meta.positions, self.rope.cos, self.rope.sin, slots,
                           cache.latent(l), cfg.kv_lora_rank, cfg.rms_eps, cfg.rope_interleaved)
        qn, qnq, qns = fused.rmsnorm(q_a, lw.q_norm, cfg.rms_eps, quant=lw.wq_b.is_fp8)
        q = linear(qn, lw.wq_b, qnq, qns).view(T, Hh, cfg.qk_head_dim)
        fused.rope_q_(q, meta.positions, self.rope.cos, self.rope.sin, cfg.qk_rope_head_dim, cfg.rope_interleaved)
        self._q, self._qn = q, qn

    def _kda(self, l: int, lw: LayerWeights, x, meta: AttnMeta, cache) -> torch.Tensor:
        """KDA layer: one stacked projection (q | k | v | output gate | low-rank decay gate | beta), the decay
        gate's second factor, the fused conv + delta-rule + gated-norm kernel over the sequence's state slot,
        then o_proj.  Heads are sharded over the TP group; the state of a sequence lives in ``cache.state``."""
        cfg, kw, tm = self.cfg, lw.kda, self.timer
        Hh, D, r = kw.heads, cfg.kda_head_dim, cfg.kda_rank
        HD = Hh * D
        with tm.timed("kda.proj", l):
            proj = linear(x, kw.w_in)
            f = linear(proj[:, 4 * HD: 4 * HD + r].contiguous(), kw.f_b)
        conv, rec = cache.state.layer(l)
        if meta.state_slots is None:
            raise RuntimeError("a model with KDA layers needs AttnMeta.state_slots")
        with tm.timed("kda.core_" + meta.mode, l):
            o = kda_ops.kda_forward(proj[:, : 3 * HD], f, proj[:, 4 * HD + r: 4 * HD + r + Hh], proj[:, 3 * HD: 4 * HD],
                                    kda_ops.KDAParams(kw.conv_w, None, kw.A_log, kw.dt_bias, kw.o_norm), conv, rec,
                                    meta.state_slots, meta.cu_seqlens if meta.mode == "prefill" else None,
                                    meta.state_has_initial if meta.mode == "prefill" else None, Hh, D, D ** -0.5,
                                    cfg.rms_eps)
        with tm.timed("attn.o_proj", l):
            return linear(o, lw.wo)

    def _side_stream(self):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def _request_parallel(self, meta: AttnMeta, T: int) -> bool:
        return (self.attn_request_parallel and meta.mode == "decode" and self.comm is not None
                and self.layout.tp_size > 1 and T % self.layout.tp_size == 0 and not self.cfg.has_dsa)

    def _mla_core_request_parallel(self, l, qbuf, meta: AttnMeta, cache):
        """Decode attention with the projections head-sharded (TP) but the core split by request: an
        all-to-all turns [all rows, my heads] queries into [my rows, all heads], each rank attends over the
        latent KV of its own rows only (the KV is not replicated: 1/world of the bytes per rank instead of
        all of them), and a second all-to-all returns [all rows, my heads] outputs for the out-absorb and
        o_proj.  Row i belongs to rank i // (T / world)."""
        W, r = self.layout.tp_size, self.layout.tp_rank
        T, Hh, D = qbuf.shape                          # [all rows, my heads, kv_lora + rope]
        L = self.cfg.kv_lora_rank
        Tl = T // W
        q = self.comm.a2a_rows_to_ranks(qbuf.view(T, Hh * D)).view(Tl, W * Hh, D)
        rows = slice(r * Tl, (r + 1) * Tl)
        o = attn_ops.mla_decode(q[..., :L], q[..., L:], cache.latent(l), meta.block_table[rows], meta.seqlens[rows],
                                self.cfg.softmax_scale, self.cfg.kv_lora_rank)
        return self.comm.a2a_ranks_to_rows(o.view(Tl, W, Hh * L)).view(T, Hh, L)

    def _mla_core(self, l, lw, q_abs, q_pe, sel, meta, cache):
        cfg = self.cfg
        if meta.mode == "decode":
            if sel is not None:
                o_lat = attn_ops.sparse_mla_decode(q_abs, q_pe, cache.latent(l), meta.block_table, sel[0], sel[1],
                                                   cfg.softmax_scale, cfg.kv_lora_rank)
            else:
                o_lat = attn_ops.mla_decode(q_abs.contiguous(), q_pe.contiguous(), cache.latent(l), meta.block_table,
                                            meta.seqlens, cfg.softmax_scale, cfg.kv_lora_rank)
        else:
            if sel is not None:
                o_lat = self._sparse_prefill(q_abs, q_pe, cache.latent(l), meta, sel)
            else:
                o_lat = attn_ops.mla_prefill(q_abs.contiguous(), q_pe.contiguous(), cache.latent(l), meta.block_table,
                                             meta.cu_seqlens, meta.ctx_lens, cfg.softmax_scale, cfg.kv_lora_rank)
            if meta.cu_seqlens[-1] < q_abs.shape[0]:
                o_lat[meta.cu_seqlens[-1]:].zero_()      # padding rows of a sequence-parallel step belong to no sequence
        return o_lat

    def _dsa_select(self, l, lw, x, qn, meta: AttnMeta, cache):
        """DSA indexer: write this step's FP8 index keys, score every cached key for each query
        (sum_h gate_h * relu(q_h . k)), keep the top-k positions.  Layers without an indexer reuse
        the selection of the nearest earlier layer that has one."""
        cfg = self.cfg
        if not cfg.layer_has_indexer(l):
            src_layer = max(i for i in cfg.indexer_full_layers if i <= l) if cfg.indexer_full_layers else l
            return meta.dsa_selection.get(src_layer)
        T = x.shape[0]
        Hi, Di = cfg.index_n_heads, cfg.index_head_dim
        rd = cfg.qk_rope_head_dim
        gpu = x.is_cuda and x.dtype == torch.bfloat16
        if gpu:
            from ..ops import dsa as dsa_ops
            gpu = dsa_ops.supported(Hi, Di, cache.page_size)
        q = linear(qn, lw.idx_wq).view(T, Hi, Di)
        gate_mul = (Hi ** -0.5) * (Di ** -0.5)
        if gpu:
            # head gates on the bf16 tensor-core GEMM (fp32 epilogue); RoPE + e4m3 + gate scaling in one kernel;
            # LayerNorm + RoPE + e4m3 + paged store of the index keys in one kernel; FP8 scores on tcgen05;
            # radix-select top-k.  Row lengths and the row -> sequence map are device tensors built once per step.
            hw = getattr(lw.idx_head_w, "_bg_bf16", None)
            if hw is None:
                hw = lw.idx_head_w.to(torch.bfloat16).contiguous()
                lw.idx_head_w._bg_bf16 = hw
            gates = gemm.bf16_gemm(x, hw, fp32_out=True)
            q8, g = dsa_ops.index_q_prepare(q, meta.positions, self.rope.cos, self.rope.sin, rd, cfg.rope_interleaved,
                                            gates, gate_mul)
            ck, cs = cache.index_keys(l)
            dsa_ops.index_k_write(linear(x, lw.idx_wk), lw.idx_k_norm_w, lw.idx_k_norm_b, meta.positions, self.rope.cos,
                                  self.rope.sin, rd, cfg.rope_interleaved, meta.slot_mapping, ck, cs)
            if meta.mode == "decode":
                lengths, bt = meta.seqlens, meta.block_table
                max_len = bt.shape[1] * cache.page_size
            else:
                lengths, bt = self._prefill_row_tables(meta, T)
                max_len = max(meta.ctx_lens[i] + meta.cu_seqlens[i + 1] - meta.cu_seqlens[i]
                              for i in range(len(meta.cu_seqlens) - 1))
            out = dsa_ops.indexer_select(q8, g, ck, cs, bt, lengths, cfg.index_topk, max_len, prepared=True)
            meta.dsa_selection[l] = out
            return out
        cos, sin = self.rope.cos[meta.positions.long()], self.rope.sin[meta.positions.long()]
        q = torch.cat([ref.apply_rope(q[..., :rd], cos, sin, cfg.rope_interleaved), q[..., rd:]], dim=-1)
        gates = (x.float() @ lw.idx_head_w.float().t()) * gate_mul
        k = ref.layernorm(linear(x, lw.idx_wk), lw.idx_k_norm_w, lw.idx_k_norm_b)
        k = torch.cat([ref.apply_rope(k[:, :rd], cos, sin, cfg.rope_interleaved), k[:, rd:]], dim=-1)
        kq, ks = ref.index_k_quant(k)
        cache.write_index_keys(l, kq, ks, meta.slot_mapping)
        idx_keys, idx_scales = cache.index_keys(l)
        P, S, _ = idx_keys.shape
        sel_idx = torch.zeros(T, cfg.index_topk, dtype=torch.int32, device=x.device)
        sel_len = torch.zeros(T, dtype=torch.int32, device=x.device)
        if meta.mode == "decode":
            lens = meta.seqlens.tolist()
            rows = [(b, b, lens[b]) for b in range(T)]
        else:
            rows = []
            for i in range(len(meta.cu_seqlens) - 1):
                a, b = meta.cu_seqlens[i], meta.cu_seqlens[i + 1]
                rows += [(t, i, meta.ctx_lens[i] + (t - a) + 1) for t in range(a, b)]
        for t, seq, L in rows:
            if L <= 0:
                continue
            if L <= cfg.index_topk:
                sel_idx[t, :L] = torch.arange(L, dtype=torch.int32, device=x.device)
                sel_len[t] = L
                continue
            npg = (L + S - 1) // S
            pages = meta.block_table[seq, :npg].long()
            kq_seq = idx_keys[pages].reshape(npg * S, Di)[:L]
            ks_seq = idx_scales[pages].reshape(npg * S)[:L]
            sc = ref.indexer_scores(q[t], gates[t], kq_seq, ks_seq)
            idx, n = ref.topk_select(sc, L, cfg.index_topk)
            sel_idx[t, :n] = idx
            sel_len[t] = n
        out = (sel_idx, sel_len)
        meta.dsa_selection[l] = out
        return out

    def _prefill_row_tables(self, meta: AttnMeta, T: int):
        """Per query row of a prefill step: (number of keys it may see, block-table row of its sequence).  Built
        once per step on the device (a row at position p sees p + 1 keys) and kept on ``meta`` for all layers."""
        if getattr(meta, "_row_tables", None) is None:
            dev = meta.positions.device
            counts = torch.tensor([meta.cu_seqlens[i + 1] - meta.cu_seqlens[i] for i in range(len(meta.cu_seqlens) - 1)],
                                  device=dev)
            row_seq = torch.repeat_interleave(torch.arange(counts.numel(), device=dev), counts)
            if row_seq.numel() < T:                      # padding rows of a sequence-parallel step: no keys
                row_seq = torch.cat([row_seq, row_seq.new_zeros(T - row_seq.numel())])
            lens = (meta.positions + 1).to(torch.int32)
            if meta.cu_seqlens[-1] < T:
                lens[meta.cu_seqlens[-1]:] = 0
            meta._row_tables = (lens.contiguous(), meta.block_table[row_seq].contiguous())
        return meta._row_tables

    def _sparse_prefill(self, q_abs, q_pe, latent, meta: AttnMeta, sel):
        """Sparse MLA for prefill rows: every query row is a one-token 'decode' over its own selection."""
        T = q_abs.shape[0]
        _, bt = self._prefill_row_tables(meta, T)
        return attn_ops.sparse_mla_decode(q_abs, q_pe, latent, bt, sel[0], sel[1], self.cfg.softmax_scale,
                                          self.cfg.kv_lora_rank)

    def _gqa(self, l: int, lw: LayerWeights, x, xq, xs, meta: AttnMeta, cache) -> torch.Tensor:
        cfg = self.cfg
        T = x.shape[0]
        D = cfg.head_dim
        Hq = lw.wo.w.shape[1] // D
        qkv = linear(x, lw.wqkv, xq, xs)
        if lw.bqkv is not None:
            qkv = qkv + lw.bqkv
        Hkv = (qkv.shape[1] // D - Hq) // 2
        q = qkv[:, : Hq * D].reshape(T, Hq, D)
        k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
        if x.is_cuda and x.dtype == torch.bfloat16 and self.rope.cos.shape[1] * 2 == D:
            # in-place RoPE kernel on the (copied, contiguous) query and key heads
            q, k = q.contiguous(), k.contiguous()
            fused.rope_q_(q, meta.positions, self.rope.cos, self.rope.sin, D, cfg.rope_interleaved)
            fused.rope_q_(k, meta.positions, self.rope.cos, self.rope.sin, D, cfg.rope_interleaved)
        else:
            cos, sin = self.rope.cos[meta.positions.long()], self.rope.sin[meta.positions.long()]
            q = ref.apply_rope(q, cos, sin, cfg.rope_interleaved)
            k = ref.apply_rope(k, cos, sin, cfg.rope_interleaved)
        kvc = cache.latent(l)                           # [P, page, 2 * Hkv_total * D]; this rank's slice is cached
        ref.kv_cache_write(kvc, torch.cat([k.reshape(T, -1), v.reshape(T, -1)], -1), meta.slot_mapping)
        window = cfg.sliding_window if (cfg.sliding_window and l % 2 == 0) else 0
        if meta.mode == "decode" and x.is_cuda:
            # paged flash-decoding kernel: lengths stay on the device (graph capturable)
            o = attn_ops.gqa_decode(q.contiguous(), kvc, meta.block_table, meta.seqlens, Hkv, cfg.softmax_scale,
                                    window=window, sinks=lw.sinks)
            return linear(o.reshape(T, -1), lw.wo)
        out = torch.zeros(T, Hq, D, dtype=x.dtype, device=x.device)
        if meta.mode == "decode":
            spans = [(b, b + 1, b, int(meta.seqlens[b]) - 1) for b in range(T)]
        else:
            spans = [(meta.cu_seqlens[i], meta.cu_seqlens[i + 1], i, meta.ctx_lens[i])
                     for i in range(len(meta.cu_seqlens) - 1)]
        for a, b, seq, ctx in spans:
            if b <= a:
                continue
            L = ctx + (b - a)
            kv = ref.gather_paged(kvc, meta.block_table[seq], L)
            ks = kv[:, : Hkv * D].reshape(L, Hkv, D)
            vs = kv[:, Hkv * D:].reshape(L, Hkv, D)
            out[a:b] = ref.gqa_attention(q[a:b], ks, vs, cfg.softmax_scale, q_start=ctx, window=window,
                                         sinks=lw.sinks)
        return linear(out.reshape(T, -1), lw.wo)

    # ------------------------------------------------------------------ feed-forward
    def _moe(self, l: int, lw: LayerWeights, x, xq, xs, meta: AttnMeta) -> torch.Tensor:
        cfg = self.cfg
        tm = self.timer
        with tm.timed("moe.router", l):
            logits = moe_ops.router_logits(x, lw.router_w)
            idx, w = moe_ops.router_topk(logits, lw.router_bias, cfg.num_experts_per_tok, cfg.n_group,
                                         cfg.topk_group, cfg.norm_topk_prob, cfg.routed_scaling_factor,
                                         cfg.scoring_func, num_valid=meta.num_valid)
        shared = None
        local = self.comm is None or self.layout.ep_size <= 1
        if (lw.w13 is not None and local and self.streamer is None and not cfg.moe_latent_size and x.is_cuda
                and self.overlap_shared_expert and meta.mode == "decode" and not tm.enabled
                and lw.experts.quant == "fp8_block" and lw.shared_gate_w is None):
            # decode on one GPU: the shared expert runs on a side stream while the routed path counts, permutes and
            # gathers its rows (small kernels that leave the GPU mostly idle); the combine adds its output, so no
            # separate add kernel either.  The router's GEMM (a split-K launch) is already queued: the side stream's
            # GEMMs are the only users of the split-K scratch until the join.
            main = torch.cuda.current_stream()
            side = self._side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared = self._mlp(x, xq, xs, lw.w13, lw.w2)
            shared.record_stream(main)
            return moe_ops.experts_forward(x, idx, w, lw.experts, 0, cfg.n_routed_experts, extra=shared,
                                           num_valid=meta.num_valid, timer=tm,
                                           before_combine=lambda: main.wait_stream(side))
        if lw.w13 is not None:
            with tm.timed("moe.shared_expert", l):
                shared = self._mlp(x, xq, xs, lw.w13, lw.w2)
            if self.comm is not None and self.layout.tp_size > 1:
                shared = self.comm.tp_reduce(shared)
            if lw.shared_gate_w is not None:
                shared = shared * torch.sigmoid(x.float() @ lw.shared_gate_w.float().t()).to(shared.dtype)
        h = x
        if cfg.moe_latent_size:
            h = linear(x, lw.latent_down)
        ew = lw.experts if self.streamer is None else self.streamer.get(l)     # streamed: blocks until the slot landed
        with tm.timed("moe.routed_experts", l):
            if self.comm is not None and self.layout.ep_size > 1:
                routed = self.comm.moe(h, idx, w, ew, cfg.n_routed_experts, num_valid=meta.num_valid)
            else:
                routed = moe_ops.experts_forward(h, idx, w, ew, 0, cfg.n_routed_experts,
                                                 num_valid=meta.num_valid, timer=tm)
        if self.streamer is not None:
            self.streamer.release(l)               # the slot returns once the kernels queued above have run
        if cfg.moe_latent_size:
            routed = linear(fused.rmsnorm(routed, lw.latent_norm, cfg.rms_eps)[0], lw.latent_up)
        return routed if shared is None else routed + shared

    # ------------------------------------------------------------------ forward
    def forward(self, ids: torch.Tensor, meta: AttnMeta, cache) -> torch.Tensor:
        """ids [T] -> fp32 logits [len(logit_rows) or T, vocab (this rank's shard under TP)]."""
        cfg = self.cfg
        h = self.w.embed[ids.long()]
        residual = None
        tp = self.comm is not None and self.layout.tp_size > 1
        for l, lw in enumerate(self.w.layers):
            fp8_in = lw.kda is None and (lw.wqkv_a or lw.wqkv).is_fp8
            tm = self.timer
            with tm.timed("norm", l):
                if residual is None:
                    residual = h.clone()
                    x, xq, xs = self._norm(h, lw.input_norm, None, fp8_in)
                else:
                    x, xq, xs = self._norm(h, lw.input_norm, residual, fp8_in)
            if lw.kda is not None:
                a = self._kda(l, lw, x, meta, cache)
            else:
                a = self._mla(l, lw, x, xq, xs, meta, cache) if cfg.is_mla else self._gqa(l, lw, x, xq, xs, meta, cache)
            if tp:
                with tm.timed("comm.tp_reduce", l):
                    a = self.comm.tp_reduce(a)
            ffn_fp8 = (lw.w13 is not None and lw.w13.is_fp8)
            with tm.timed("norm", l):
                x, xq, xs = self._norm(a, lw.post_norm, residual, ffn_fp8)
            if cfg.is_moe_layer(l):
                h = self._moe(l, lw, x, xq, xs, meta)
            else:
                with tm.timed("dense_mlp", l):
                    h = self._mlp(x, xq, xs, lw.w13, lw.w2)
                if tp:
                    with tm.timed("comm.tp_reduce", l):
                        h = self.comm.tp_reduce(h)
        x, _, _ = self._norm(h, self.w.final_norm, residual, False)
        if meta.logit_rows is not None:
            x = x[meta.logit_rows.long()]
        with self.timer.timed("lm_head"):
            logits = self._lm_head(x)
        if tp:
            logits = self.comm.tp_gather_vocab(logits)
        if self.streamer is not None:
            self.streamer.end_step()
        return logits

    # ------------------------------------------------------------------ sequence-parallel forward
    @staticmethod
    def supports_sequence_parallel(cfg: ModelConfig) -> Optional[str]:
        """``None`` when ``forward_sp`` (fused NVLink kernels) can run ``cfg``, otherwise the reason it cannot."""
        if cfg.is_v4:
            return "DeepSeek-V4 attention is replicated inside an engine; its experts use the collective baseline"
        if not cfg.is_mla:
            return "GQA attention runs tensor-parallel through forward() and the collective baseline"
        if cfg.has_kda:
            return "KDA layers run tensor-parallel through forward() and the collective baseline"
        if cfg.has_dsa:
            return "DSA indexer layers need the full-width hidden rows: they run through forward() and the collective baseline"
        if cfg.quant != "fp8_block":
            return "the fused kernels move block-scaled FP8 rows; other expert formats use the collective baseline"
        if cfg.moe_latent_size:
            return "latent-MoE projections are not part of the fused path"
        if cfg.shared_expert_gate:
            return "the gated shared expert is not part of the fused path"
        if cfg.hidden_size % 128 or cfg.expert_hidden % 128:
            return "hidden sizes must be multiples of the 128-wide quantisation block"
        return None

    def forward_sp(self, ids: torch.Tensor, meta: AttnMeta, cache) -> torch.Tensor:
        """Tensor-parallel attention + expert-parallel MoE with a row-sharded residual stream and the
        collectives fused into the kernels (``parallel.fused.FusedComm``).  ``ids`` holds all T tokens of
        the step (T divisible by the world size); returns fp32 logits of this rank's own rows
        [T / world, vocab] (rows rank*Tl .. (rank+1)*Tl)."""
        cfg, comm, tm = self.cfg, self.comm, self.timer
        if cfg.has_kda or not cfg.is_mla:
            raise NotImplementedError("the fused sequence-parallel path covers MLA layers; models with KDA or GQA "
                                      "layers run tensor-parallel through forward() and the collective baseline")
        W, r = comm.world, comm.rank
        T = ids.shape[0]
        assert T % W == 0, "pad the step to a multiple of the world size"
        Tl = T // W
        eps = cfg.rms_eps
        comm.begin_step()
        src = self.w.embed[ids[r * Tl:(r + 1) * Tl].long()]      # local rows of the residual stream
        residual = torch.empty_like(src)
        first = True
        nv_local = None
        if meta.num_valid is not None:                           # padding rows of a graph bucket
            nv_local = (meta.num_valid - r * Tl).clamp(0, Tl).to(torch.int32)
        for l, lw in enumerate(self.w.layers):
            # input norm of own rows (+ previous sublayer's output), quantised rows pushed to every rank
            with tm.timed("sp.norm_push", l):
                comm.sp_norm_push(src, residual, lw.input_norm, eps, from_rs=src is None, has_residual=not first,
                                  push=True, want_y=False, want_q=False)
            first = False
            with tm.timed("attn.qkv_a_gemm", l):
                qkv_a = comm.ag_gemm(lw.wqkv_a, T)
            o = self._mla_from_qkv_a(l, lw, qkv_a, None, meta, cache)
            with tm.timed("attn.o_proj_rs", l):
                oq, os_ = fused.act_quant(o)
                comm.gemm_rs(oq, os_, lw.wo, T)
            if cfg.is_moe_layer(l):
                with tm.timed("sp.norm_push", l):
                    x, xq, xs = comm.sp_norm_push(None, residual, lw.post_norm, eps, from_rs=True, has_residual=True,
                                                  push=False)
                with tm.timed("moe.router", l):
                    logits = moe_ops.router_logits(x, lw.router_w)
                    idx, w = moe_ops.router_topk(logits, lw.router_bias, cfg.num_experts_per_tok, cfg.n_group,
                                                 cfg.topk_group, cfg.norm_topk_prob, cfg.routed_scaling_factor,
                                                 cfg.scoring_func, num_valid=nv_local)
                shared, join = None, None
                if lw.w13 is not None:
                    if self.overlap_shared_expert and x.is_cuda and meta.mode == "decode" and not tm.enabled:
                        # decode: the shared expert (weight streaming) runs on a side stream under the dispatch
                        # chain (counts -> layout -> send: one-CTA kernels and peer handshakes that leave the GPU
                        # idle); the combine, which adds its output, waits for it.  Safe with the split-K scratch:
                        # at these sizes both of its GEMMs are swapped-operand launches, which do not use it.
                        main = torch.cuda.current_stream()
                        side = self._side_stream()
                        side.wait_stream(main)
                        with torch.cuda.stream(side):
                            shared = self._mlp(x, xq, xs, lw.w13, lw.w2)
                        shared.record_stream(main)
                        join = lambda: main.wait_stream(side)      # noqa: E731
                    else:
                        with tm.timed("moe.shared_expert", l):
                            shared = self._mlp(x, xq, xs, lw.w13, lw.w2)
                with tm.timed("moe.routed_experts", l):
                    src = comm.moe_sp(x, idx, w, lw.experts, extra=shared, timer=self.timer, before_combine=join)
            else:
                with tm.timed("sp.norm_push", l):
                    comm.sp_norm_push(None, residual, lw.post_norm, eps, from_rs=True, has_residual=True, push=True,
                                      want_y=False, want_q=False)
                with tm.timed("dense_mlp", l):
                    act = comm.ag_gemm(lw.w13, T, silu_mul=True)
                    aq, as_ = fused.act_quant(act)
                    comm.gemm_rs(aq, as_, lw.w2, T)
                src = None                                       # next norm sums the reduce-scatter partials
        x, _, _ = comm.sp_norm_push(src, residual, self.w.final_norm, eps, from_rs=src is None, has_residual=True,
                                    push=False, want_q=False)
        comm.end_step()
        if meta.logit_rows is not None:
            # only the wanted rows that this rank owns (the caller gathers them in rank order)
            rows = meta.logit_rows.long()
            x = x[rows[(rows >= r * Tl) & (rows < (r + 1) * Tl)] - r * Tl]
        with tm.timed("lm_head"):
            return self._lm_head(x)
