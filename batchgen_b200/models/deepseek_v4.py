"""DeepSeek-V4 (Flash / Pro): hyper-connection residual streams, one latent KV head shared by all query heads
(K = V), a sliding window of raw KV rows plus pooled ("compressed") entries, a top-k indexer over the pooled entries
on ratio-4 layers, a grouped low-rank output projection, and a MoE whose first layers route by token id.

How the state is kept here:

* per sequence (a slot of ``runtime.kv_cache.V4StatePool``): each layer's ring of the last ``window`` KV rows, and
  on compressed layers the projections and gate scores of the tokens that are not pooled yet;
* paged (``PagedKVCache.v4_comp`` / ``v4_idx``): the pooled entries.  Entry c of a ratio-r layer covers tokens
  c*r .. c*r + r - 1 and lives in the page of its first token, so the engine's page allocator and block tables
  serve this family unchanged.

The compressor is written over absolute positions, so one routine serves a whole prompt, a prefill chunk that
continues a sequence, and a decode step (a chunk of one token): pending rows of the open window come from the
sequence's state, complete windows are pooled and written to their pages, the rest goes back to the state.
Decode steps take a second route that handles every row of the batch in the same tensor operations and reads nothing
back to the host (``_attention_decode``): lengths, ring rows, window closings and entry slots are all computed from
the position tensor.

Pooling of window j (ratio r, width d): softmax over the r tokens of (w_gate x_t + ape[t mod r]), per dimension,
weights the rows w_kv x_t.  With overlapped windows (ratio 4) the projections are 2d wide: a window pools its own
tokens through the upper half and the previous window's tokens through the lower half (2r rows in one softmax).
The pooled row is RMS-normalised and rotated (last ``rope`` dims) at the position of the window's first token.

Attention of the query at position p: keys = the raw rows at positions (p - window, p] and the pooled entries
c < (p + 1) // r (on ratio-4 layers only the ``index_topk`` best by the indexer's score
sum_h w_h relu(q_h . k_c)); one softmax over both sets with a per-head sink logit in the denominator; values are
the same rows; the output's rope dims are rotated back before the grouped output projection.

The indexer's Hadamard rotation and FP4 / FP8 quantisation-aware rounding of cached rows are left out: the rotation
is orthogonal (scores do not change) and the rounding only simulates training-time noise.

Parallelism: attention is replicated inside an engine (data-parallel cohorts come from the server's ``--dp-size``
front); routed experts are expert-parallel through ``comm.moe`` when a communicator is attached.

Reference parity: batchgen/models/deepseek/deepseekv4_flash/model.py (module surface, fallback attention :349-420,
gate :433-489, hyper-connections :588-700) and its config (config.py:36-119); the compressed attention follows the
model definition the reference vendors beside it (assets/inference/model.py: Compressor, Indexer, Attention).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import fused, ref
from ..ops import moe as moe_ops
from ..ops.moe import ExpertWeights
from ..utils.timing import null_timer
from .transformer import AttnMeta, linear
from .weights import Linear, ParallelLayout, WeightSource, make_linear


@dataclass
class CompressorWeights:
    wkv: torch.Tensor = None     # [c * d, H] fp32 (pooling runs in fp32)
    wgate: torch.Tensor = None   # [c * d, H] fp32
    ape: torch.Tensor = None     # [r, c * d] fp32: per-slot score offset
    norm: torch.Tensor = None    # [d]
    ratio: int = 0
    width: int = 0               # d

    @property
    def overlap(self) -> bool:
        return self.ratio == 4


@dataclass
class V4LayerWeights:
    attn_norm: torch.Tensor = None
    ffn_norm: torch.Tensor = None
    hc_attn: Tuple[torch.Tensor, torch.Tensor, torch.Tensor] = None   # (fn [(2 + hc) hc, hc H], base, scale[3]) fp32
    hc_ffn: Tuple[torch.Tensor, torch.Tensor, torch.Tensor] = None
    wq_a: Linear = None
    q_norm: torch.Tensor = None
    wq_b: Linear = None
    wkv: Linear = None
    kv_norm: torch.Tensor = None
    wo_a: List[Linear] = field(default_factory=list)   # per group [o_lora, heads / groups * D]
    wo_b: Linear = None
    sink: torch.Tensor = None                          # [heads] fp32
    comp: Optional[CompressorWeights] = None
    idx_wq: Linear = None                              # [Hi * Di, q_lora]
    idx_wproj: torch.Tensor = None                     # [Hi, H]
    idx_comp: Optional[CompressorWeights] = None
    router_w: torch.Tensor = None
    router_bias: torch.Tensor = None
    tid2eid: torch.Tensor = None                       # [vocab, k] int64 (hash-routed layers)
    experts: ExpertWeights = None
    w13: Linear = None                                 # shared expert
    w2: Linear = None


@dataclass
class V4Weights:
    embed: torch.Tensor = None
    final_norm: torch.Tensor = None
    lm_head: torch.Tensor = None
    hc_head: Tuple[torch.Tensor, torch.Tensor, torch.Tensor] = None    # (fn [hc, hc H], base [hc], scale [1])
    layers: List[V4LayerWeights] = field(default_factory=list)


def _compressor(src: WeightSource, prefix: str, H: int, ratio: int, width: int, dtype) -> CompressorWeights:
    c = 2 if ratio == 4 else 1
    return CompressorWeights(wkv=src.get(f"{prefix}.wkv.weight", (c * width, H)).float(),
                             wgate=src.get(f"{prefix}.wgate.weight", (c * width, H)).float(),
                             ape=src.get(f"{prefix}.ape", (ratio, c * width), "bias").float(),
                             norm=src.get(f"{prefix}.norm.weight", (width,), "norm").to(dtype), ratio=ratio, width=width)


def _hc(src: WeightSource, prefix: str, rows: int, cols: int, n_scale: int):
    return (src.get(f"{prefix}_fn", (rows, cols)).float(), src.get(f"{prefix}_base", (rows,), "bias").float(),
            src.get(f"{prefix}_scale", (n_scale,), "norm").float())


def build_v4_weights(cfg: ModelConfig, layout: ParallelLayout, src: WeightSource, dtype: torch.dtype) -> V4Weights:
    """Tensor names follow the published checkpoint (``layers.L.attn.wq_a.weight`` ...)."""
    H, D, Hh, hc = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.hc_mult
    quant = "none" if cfg.quant == "none" else "fp8_block"      # attention / shared-expert linears; experts: cfg.quant
    w = V4Weights()
    w.embed = src.get("embed.weight", (cfg.vocab_size, H)).to(dtype)
    w.final_norm = src.get("norm.weight", (H,), "norm").to(dtype)
    w.lm_head = src.get("head.weight", (cfg.vocab_size, H)).to(dtype)
    w.hc_head = _hc(src, "hc_head", hc, hc * H, 1)
    mix = (2 + hc) * hc
    G, R = cfg.o_groups, cfg.o_lora_rank
    for l, ratio in enumerate(cfg.compress_ratios):
        p, a, f = f"layers.{l}", f"layers.{l}.attn", f"layers.{l}.ffn"
        lw = V4LayerWeights()
        lw.attn_norm = src.get(f"{p}.attn_norm.weight", (H,), "norm").to(dtype)
        lw.ffn_norm = src.get(f"{p}.ffn_norm.weight", (H,), "norm").to(dtype)
        lw.hc_attn = _hc(src, f"{p}.hc_attn", mix, hc * H, 3)
        lw.hc_ffn = _hc(src, f"{p}.hc_ffn", mix, hc * H, 3)
        lw.wq_a = make_linear(src.get(f"{a}.wq_a.weight", (cfg.q_lora_rank, H)), quant, dtype)
        lw.q_norm = src.get(f"{a}.q_norm.weight", (cfg.q_lora_rank,), "norm").to(dtype)
        lw.wq_b = make_linear(src.get(f"{a}.wq_b.weight", (Hh * D, cfg.q_lora_rank)), quant, dtype)
        lw.wkv = make_linear(src.get(f"{a}.wkv.weight", (D, H)), quant, dtype)
        lw.kv_norm = src.get(f"{a}.kv_norm.weight", (D,), "norm").to(dtype)
        wo_a = src.get(f"{a}.wo_a.weight", (G * R, Hh * D // G)).view(G, R, Hh * D // G)
        lw.wo_a = [make_linear(wo_a[g].contiguous(), "none", dtype) for g in range(G)]
        lw.wo_b = make_linear(src.get(f"{a}.wo_b.weight", (H, G * R)), quant, dtype)
        lw.sink = src.get(f"{a}.attn_sink", (Hh,), "bias").float()
        if ratio:
            lw.comp = _compressor(src, f"{a}.compressor", H, ratio, D, dtype)
            if ratio == 4:
                Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                lw.idx_wq = make_linear(src.get(f"{a}.indexer.wq_b.weight", (Hi * Di, cfg.q_lora_rank)), "none", dtype)
                lw.idx_wproj = src.get(f"{a}.indexer.weights_proj.weight", (Hi, H)).to(dtype)
                lw.idx_comp = _compressor(src, f"{a}.indexer.compressor", H, ratio, Di, dtype)
        E, I, K = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.num_experts_per_tok
        lw.router_w = src.get(f"{f}.gate.weight", (E, H)).float()
        if l < cfg.num_hash_layers:
            # a fixed table token id -> its K experts (distinct per token): read from the checkpoint when a loader
            # has it ([vocab, K] integers), otherwise drawn from the seeded source
            table = src.loader(f"{f}.gate.tid2eid", (cfg.vocab_size, K)) if src.loader is not None else None
            if table is not None:
                lw.tid2eid = table.to(src.device, torch.int64)
            else:
                lw.tid2eid = src.get(f"{f}.gate.tid2eid", (cfg.vocab_size, E)).topk(K, dim=-1)[1]
        else:
            lw.router_bias = src.get(f"{f}.gate.bias", (E,), "bias").float()
        e0, e1 = layout.expert_range(E)
        w13s, w2s, s13, s2 = [], [], [], []
        w4 = cfg.quant in ("mxfp4", "int4") and H % 64 == 0 and I % 64 == 0
        for e in range(e0, e1):
            ep = f"{f}.experts.{e}"
            gu = torch.cat([src.get(f"{ep}.w1.weight", (I, H)), src.get(f"{ep}.w3.weight", (I, H))], 0)
            dn = src.get(f"{ep}.w2.weight", (H, I))
            if w4:
                if cfg.quant == "mxfp4":
                    from ..ops.mxfp4 import quantize as quantize_w4
                else:
                    from ..ops.int4 import quantize as quantize_w4
                (q13, sc13), (q2, sc2) = quantize_w4(gu), quantize_w4(dn)
                w13s.append(q13); s13.append(sc13); w2s.append(q2); s2.append(sc2)
            else:
                w13s.append(gu.to(dtype)); w2s.append(dn.to(dtype))
        lw.experts = ExpertWeights(w13=torch.stack(w13s), w2=torch.stack(w2s),
                                   w13_s=torch.stack(s13) if s13 else None, w2_s=torch.stack(s2) if s2 else None,
                                   quant=cfg.quant if w4 else "none", activation="silu_limit",
                                   act_limit=cfg.swiglu_limit).to_device_layout()
        sp = f"{f}.shared_experts"
        lw.w13 = make_linear(torch.cat([src.get(f"{sp}.w1.weight", (I, H)), src.get(f"{sp}.w3.weight", (I, H))], 0),
                             quant, dtype).interleave_gate_up_()
        lw.w2 = make_linear(src.get(f"{sp}.w2.weight", (H, I)), quant, dtype)
        w.layers.append(lw)
    return w


def hc_split(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, hc: int, iters: int, eps: float):
    """mixes [T, (2 + hc) hc] -> pre [T, hc], post [T, hc], comb [T, hc, hc] (Sinkhorn-normalised)."""
    pre = torch.sigmoid(mixes[:, :hc] * scale[0] + base[:hc]) + eps
    post = 2 * torch.sigmoid(mixes[:, hc: 2 * hc] * scale[1] + base[hc: 2 * hc])
    comb = mixes[:, 2 * hc:].view(-1, hc, hc) * scale[2] + base[2 * hc:].view(hc, hc)
    comb = torch.softmax(comb, dim=-1) + eps
    comb = comb / (comb.sum(dim=-2, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        comb = comb / (comb.sum(dim=-1, keepdim=True) + eps)
        comb = comb / (comb.sum(dim=-2, keepdim=True) + eps)
    return pre, post, comb


def pool_windows(kv: torch.Tensor, sc: torch.Tensor, ctx: int, cw: CompressorWeights, pend_kv: torch.Tensor,
                 pend_sc: torch.Tensor) -> torch.Tensor:
    """Pool the windows that the tokens at positions ctx .. ctx + n - 1 complete.

    kv / sc: [n, c d] fp32 projections of the new tokens (scores without the slot offset).  ``pend_kv`` /
    ``pend_sc`` [c r, c d] is the sequence's state and is updated in place: rows [off, off + ctx % r) hold the
    open window's tokens, and with overlapped windows rows [0, r) hold the last complete window (scores -inf before
    the first one).  Returns the pooled rows [m, d] of windows ctx // r .. ctx // r + m - 1 (before norm / rope)."""
    r, d, n = cw.ratio, cw.width, kv.shape[0]
    off = r if cw.overlap else 0
    k0 = ctx % r
    slots = (ctx + torch.arange(n, device=kv.device)) % r
    cur_kv = torch.cat([pend_kv[off: off + k0], kv], 0)
    cur_sc = torch.cat([pend_sc[off: off + k0], sc + cw.ape[slots]], 0)
    m = (k0 + n) // r
    rem = k0 + n - m * r
    pooled = kv.new_zeros(0, d)
    if m:
        wk = cur_kv[: m * r].view(m, r, -1)
        ws = cur_sc[: m * r].view(m, r, -1)
        if cw.overlap:
            prev_k = torch.cat([pend_kv[:r].unsqueeze(0), wk[:-1]], 0)
            prev_s = torch.cat([pend_sc[:r].unsqueeze(0), ws[:-1]], 0)
            rows = torch.cat([prev_k[..., :d], wk[..., d:]], 1)                  # [m, 2r, d]
            gate = torch.cat([prev_s[..., :d], ws[..., d:]], 1)
            last_k, last_s = wk[-1].clone(), ws[-1].clone()
        else:
            rows, gate = wk, ws
        pooled = (rows * torch.softmax(gate, dim=1)).sum(1)
        if cw.overlap:
            pend_kv[:r] = last_k
            pend_sc[:r] = last_s
    tail_k, tail_s = cur_kv[m * r:].clone(), cur_sc[m * r:].clone()
    pend_kv[off: off + rem] = tail_k
    pend_sc[off: off + rem] = tail_s
    return pooled


class DeepSeekV4:
    """Same calling contract as ``Transformer``: ``forward(ids [T], meta, cache) -> fp32 logits``."""

    def __init__(self, cfg: ModelConfig, weights: V4Weights, layout: Optional[ParallelLayout] = None, comm=None,
                 max_positions: int = 8192):
        assert cfg.is_v4
        self.cfg, self.w, self.comm = cfg, weights, comm
        self.layout = layout or ParallelLayout()
        self.device, self.dtype = weights.embed.device, weights.embed.dtype
        self.timer = null_timer()
        self.attn_request_parallel = False
        self.streamer = None
        self.batched_decode = True     # decode steps run all rows at once without host reads (False: row by row)
        self.kernel_decode = True      # 512-wide heads on the GPU: the decode core runs on the absorbed-MLA kernel
        self.kernel_math_anywhere = False   # tests: take that route on any device / geometry (reference MLA math)
        rd = cfg.qk_rope_head_dim
        pos = torch.arange(max_positions, dtype=torch.float32)
        # compressed layers rotate with their own base and YaRN; window-only layers with the plain base
        inv_c = ref.rope_inv_freq(rd, cfg.compress_rope_theta or cfg.rope_theta, cfg.rope_scaling_factor,
                                  cfg.rope_original_max_pos, cfg.rope_beta_fast, cfg.rope_beta_slow)
        inv_w = ref.rope_inv_freq(rd, cfg.rope_theta)
        self._rope = {True: tuple(t.to(self.device) for t in ((pos[:, None] * inv_c).cos(), (pos[:, None] * inv_c).sin())),
                      False: tuple(t.to(self.device) for t in ((pos[:, None] * inv_w).cos(), (pos[:, None] * inv_w).sin()))}
        self.max_positions = max_positions

    # ------------------------------------------------------------------ helpers
    def _rms(self, x, w):
        return fused.rmsnorm(x, w, self.cfg.rms_eps)[0]

    def _rotate(self, x, positions, compressed: bool, inverse: bool = False):
        """Rotate the last ``rope`` dims of x [n, ..., D] by the angles of ``positions`` [n]."""
        rd = self.cfg.qk_rope_head_dim
        cos, sin = self._rope[compressed]
        cos, sin = cos[positions.long()], sin[positions.long()]
        tail = ref.apply_rope(x[..., -rd:], cos, -sin if inverse else sin, True)
        return torch.cat([x[..., :-rd], tail], -1)

    def _hc_pre(self, h, hcw):
        """h [T, hc, H] -> (mixed [T, H], post [T, hc], comb [T, hc, hc])."""
        cfg = self.cfg
        fn, base, scale = hcw
        flat = h.reshape(h.shape[0], -1).float()
        rs = torch.rsqrt(flat.square().mean(-1, keepdim=True) + cfg.rms_eps)
        pre, post, comb = hc_split((flat @ fn.t()) * rs, scale, base, cfg.hc_mult, cfg.hc_sinkhorn_iters, cfg.hc_eps)
        return (pre.unsqueeze(-1) * h.float()).sum(1).to(h.dtype), post, comb

    @staticmethod
    def _hc_post(out, residual, post, comb):
        """new[j] = post[j] * out + sum_i comb[i, j] * residual[i]."""
        y = post.unsqueeze(-1) * out.float().unsqueeze(1) + torch.einsum("tij,tih->tjh", comb, residual.float())
        return y.to(out.dtype)

    def _spans(self, meta: AttnMeta, T: int):
        """(first row, end row, sequence, tokens cached before) of every sequence of the step."""
        if meta.mode == "decode":
            lens = meta.seqlens.tolist()
            return [(b, b + 1, b, int(lens[b]) - 1) for b in range(T)]
        return [(meta.cu_seqlens[i], meta.cu_seqlens[i + 1], i, meta.ctx_lens[i]) for i in range(len(meta.cu_seqlens) - 1)]

    # ------------------------------------------------------------------ compressed entries
    def _entry_slots(self, block_row: torch.Tensor, first: int, count: int, ratio: int, epp: int, page_size: int):
        """Flat (page * epp + slot) index of entries first .. first + count - 1 of one sequence."""
        c = torch.arange(first, first + count, device=block_row.device)
        tok = c * ratio
        return block_row[(tok // page_size).long()].long() * epp + (tok % page_size) // ratio

    def _compress(self, cw: CompressorWeights, x, ctx: int, pend_kv, pend_sc, pool: torch.Tensor, block_row, page_size: int):
        """Project, pool and store the entries completed by a chunk; returns how many entries the sequence has now."""
        n = x.shape[0]
        xf = x.float()
        if ctx == 0:
            pend_kv.zero_()
            pend_sc.zero_()
            if cw.overlap:
                pend_sc[: cw.ratio] = float("-inf")
        pooled = pool_windows(xf @ cw.wkv.t(), xf @ cw.wgate.t(), ctx, cw, pend_kv, pend_sc)
        m = pooled.shape[0]
        if m:
            first = ctx // cw.ratio
            rows = self._rms(pooled.to(pool.dtype), cw.norm)
            firsts = (first + torch.arange(m, device=x.device)) * cw.ratio
            rows = self._rotate(rows, firsts, True)
            epp = pool.shape[1]
            pool.view(-1, pool.shape[-1])[self._entry_slots(block_row, first, m, cw.ratio, epp, page_size)] = rows.to(pool.dtype)
        return (ctx + n) // cw.ratio

    # ------------------------------------------------------------------ decode: all rows at once, no host reads
    def _compress_step(self, cw: CompressorWeights, x, pos, slots, valid, P_kv, P_sc, pool, block_table, page_size: int):
        """One decode token per row: park its projections in the open window, pool the rows whose window closes and
        store their entry.  ``P_kv`` / ``P_sc`` are the state parts of every slot ([slots + 1, c r, c d]).  Rows whose
        window stays open write a scratch value into the entry that is still in progress (nobody reads it before the
        closing step overwrites it), and rows without a sequence use the scratch slot and the scratch page, so the
        routine needs no row selection on the host and never writes one place from two rows."""
        r, d = cw.ratio, cw.width
        off = r if cw.overlap else 0
        xf = x.float()
        k0 = (pos % r).long()
        row = off + k0
        P_kv[slots, row] = xf @ cw.wkv.t()
        P_sc[slots, row] = xf @ cw.wgate.t() + cw.ape[k0]
        S_kv, S_sc = P_kv[slots], P_sc[slots]                                   # [B, c r, c d]
        if cw.overlap:
            rows = torch.cat([S_kv[:, :r, :d], S_kv[:, r:, d:]], 1)
            gate = torch.cat([S_sc[:, :r, :d], S_sc[:, r:, d:]], 1)
        else:
            rows, gate = S_kv, S_sc
        pooled = torch.nan_to_num((rows * torch.softmax(gate, dim=1)).sum(1))    # open windows may pool stale scores
        c = (pos // r).long()
        ent = self._rotate(self._rms(pooled.to(pool.dtype), cw.norm), c * r, True)
        epp = pool.shape[1]
        tok = c * r
        page = block_table[torch.arange(len(c), device=x.device), (tok // page_size)].long()
        page = torch.where(valid, page, torch.full_like(page, pool.shape[0] - 1))
        pool.view(-1, pool.shape[-1])[page * epp + (tok % page_size) // r] = ent.to(pool.dtype)
        if cw.overlap:
            cm = (((pos + 1) % r) == 0).view(-1, 1, 1)
            P_kv[slots, :r] = torch.where(cm, S_kv[:, r:], S_kv[:, :r])
            P_sc[slots, :r] = torch.where(cm, S_sc[:, r:], S_sc[:, :r])
        return (pos + 1) // r

    def _attention_decode(self, l: int, lw: V4LayerWeights, x, meta: AttnMeta, cache, q, kv, qi, wi) -> torch.Tensor:
        cfg = self.cfg
        B, D, Hh, win = x.shape[0], cfg.head_dim, cfg.num_heads, cfg.sliding_window
        ratio = cfg.compress_ratios[l]
        ps = cache.page_size
        dev = x.device
        pos = meta.positions.long()
        valid = meta.state_slots >= 0
        rec = cache.state.rec[0]
        slots = torch.where(valid, meta.state_slots, torch.full_like(meta.state_slots, rec.shape[0] - 1)).long()

        def part(name):
            off, shape = cache.state.offsets[(l, name)]
            return rec[:, off: off + shape[0] * shape[1]].view(rec.shape[0], *shape)

        R = part("ring")
        j = (pos % win)
        R[slots, j] = kv.float()
        ring = R[slots]                                                          # [B, win, D]
        jj = torch.arange(win, device=dev)
        held = pos[:, None] - ((pos[:, None] - jj[None, :]) % win)               # position each ring row holds
        keys, mask = ring, held >= 0
        if ratio:
            bt = meta.block_table
            pool = cache.v4_comp[l]
            E = self._compress_step(lw.comp, x, pos, slots, valid, part("kv"), part("score"), pool, bt, ps)
            Emax = max(1, bt.shape[1] * ps // ratio)
            c = torch.arange(Emax, device=dev)
            tok = c * ratio
            col = (tok // ps).clamp_max(bt.shape[1] - 1)
            flat = bt[:, col].long() * pool.shape[1] + ((tok % ps) // ratio)[None, :]
            ent = pool.view(-1, D)[flat].float()                                 # [B, Emax, D]
            visible = c[None, :] < E[:, None]
            if lw.idx_comp is not None:
                ipool = cache.v4_idx[l]
                self._compress_step(lw.idx_comp, x, pos, slots, valid, part("idx_kv"), part("idx_score"), ipool, bt, ps)
                if Emax > cfg.index_topk:
                    ik = ipool.view(-1, ipool.shape[-1])[flat].float()
                    sc = (torch.relu(torch.einsum("bhd,bed->bhe", qi, ik)) * wi.unsqueeze(-1)).sum(1)
                    sc = sc.masked_fill(~visible, float("-inf"))
                    top = sc.topk(cfg.index_topk, dim=-1)[1]
                    visible = visible & torch.zeros_like(visible).scatter_(1, top, True)
            keys = torch.cat([keys, ent], 1)
            mask = torch.cat([mask, visible], 1)
        if self.kernel_decode and (self.kernel_math_anywhere or (x.is_cuda and D == 512 and self.dtype == torch.bfloat16
                                                                and Hh % 8 == 0)):
            out = self._decode_core_on_mla_kernel(q, keys, mask, lw.sink)
        else:
            s = torch.einsum("bhd,bkd->bhk", q, keys) * D ** -0.5
            s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
            sink = lw.sink.view(1, Hh, 1).expand(B, Hh, 1)
            p = torch.softmax(torch.cat([s, sink], -1), -1)[..., :-1]
            out = torch.einsum("bhk,bkd->bhd", p, keys)
        return torch.where(valid.view(-1, 1, 1), out, torch.zeros_like(out))

    def _decode_core_on_mla_kernel(self, q, keys, mask, sink) -> torch.Tensor:
        """The decode attention core on the absorbed-MLA decode kernel (tcgen05, 512-wide latent rows with 64 extra
        score-only columns).  K = V = the gathered rows; the 64 extra columns, which carry the rotary part for MLA
        models, carry flags here: column 0 is 1 on one appended row whose value part is zero and whose score is the
        head's sink logit (the query's column 0 holds sink / scale), so the sink joins the softmax denominator only;
        column 1 holds a large negative number on masked rows (ring rows not written yet, entries that are not visible
        or not selected), and the query's column 1 is 1, so those rows get zero weight.  Every row of the batch then has
        the same length and nothing is compacted."""
        from ..ops import attention as attn_ops
        B, Hh, D = q.shape
        dev = q.device
        dt = self.dtype
        Kk = keys.shape[1]
        page = 64
        K = (Kk + 1 + page - 1) // page * page
        scale = D ** -0.5
        dense = torch.zeros(B, K, D + 64, dtype=dt, device=dev)
        dense[:, :Kk, :D] = torch.where(mask.unsqueeze(-1), keys, torch.zeros_like(keys)).to(dt)
        dense[:, :Kk, D + 1] = torch.where(mask, 0.0, -30000.0 / scale).to(dt)
        dense[:, Kk, D] = 1.0
        q_pe = torch.zeros(B, Hh, 64, dtype=dt, device=dev)
        q_pe[:, :, 0] = (sink / scale).to(dt)
        q_pe[:, :, 1] = 1.0
        lens = torch.full((B,), Kk + 1, dtype=torch.int32, device=dev)
        bt = torch.arange(B * (K // page), dtype=torch.int32, device=dev).view(B, K // page)
        out = attn_ops.mla_decode(q.to(dt).contiguous(), q_pe, dense.view(B * (K // page), page, D + 64), bt, lens, scale, D)
        return out.float()

    # ------------------------------------------------------------------ attention
    def _attention(self, l: int, lw: V4LayerWeights, x, meta: AttnMeta, cache) -> torch.Tensor:
        cfg = self.cfg
        T, D, Hh, win = x.shape[0], cfg.head_dim, cfg.num_heads, cfg.sliding_window
        ratio = cfg.compress_ratios[l]
        compressed = ratio > 0
        if meta.state_slots is None:
            raise RuntimeError("a DeepSeek-V4 model needs AttnMeta.state_slots (window and compressor state per sequence)")
        qr = self._rms(linear(x, lw.wq_a), lw.q_norm)
        q = linear(qr, lw.wq_b).view(T, Hh, D).float()
        q = q * torch.rsqrt(q.square().mean(-1, keepdim=True) + cfg.rms_eps)
        q = self._rotate(q, meta.positions, compressed)
        kv = self._rotate(self._rms(linear(x, lw.wkv), lw.kv_norm), meta.positions, compressed)        # [T, D]
        if lw.idx_wq is not None:
            Hi, Di = cfg.index_n_heads, cfg.index_head_dim
            qi = self._rotate(linear(qr, lw.idx_wq).view(T, Hi, Di).float(), meta.positions, True)
            wi = (x.float() @ lw.idx_wproj.float().t()) * (Di ** -0.5 * Hi ** -0.5)                 # [T, Hi]
        if meta.mode == "decode" and self.batched_decode:
            out = self._attention_decode(l, lw, x, meta, cache, q, kv, qi if lw.idx_wq is not None else None,
                                         wi if lw.idx_wq is not None else None)
            return self._project_out(lw, out, meta, compressed)
        out = torch.zeros(T, Hh, D, dtype=torch.float32, device=x.device)
        slots = meta.state_slots.tolist()
        ps = cache.page_size
        scale = D ** -0.5
        for a, b, seq, ctx in self._spans(meta, T):
            slot = slots[seq]
            if b <= a or slot < 0:
                continue
            n = b - a
            ring = cache.state.view(slot, l, "ring")
            # raw rows visible to the chunk: up to window - 1 cached positions, then the chunk itself
            m0 = min(ctx, win - 1)
            old_pos = torch.arange(ctx - m0, ctx, device=x.device)
            keys = torch.cat([ring[(old_pos % win).long()], kv[a:b].float()], 0)
            kpos = torch.cat([old_pos, torch.arange(ctx, ctx + n, device=x.device)])
            keep = min(n, win)
            new_pos = torch.arange(ctx + n - keep, ctx + n, device=x.device)
            ring[(new_pos % win).long()] = kv[b - keep: b].float()
            qpos = torch.arange(ctx, ctx + n, device=x.device)
            mask = (kpos[None, :] <= qpos[:, None]) & (kpos[None, :] > qpos[:, None] - win)          # [n, K_w]
            if compressed:
                brow = meta.block_table[seq]
                pool = cache.v4_comp[l]
                E = self._compress(lw.comp, x[a:b], ctx, cache.state.view(slot, l, "kv"), cache.state.view(slot, l, "score"),
                                   pool, brow, ps)
                if E:
                    ent = pool.view(-1, D)[self._entry_slots(brow, 0, E, ratio, pool.shape[1], ps)].float()
                    visible = torch.arange(E, device=x.device)[None, :] < ((qpos + 1) // ratio)[:, None]   # [n, E]
                else:
                    ent, visible = keys.new_zeros(0, D), mask.new_zeros(n, 0)
                if lw.idx_comp is not None:
                    ipool = cache.v4_idx[l]
                    self._compress(lw.idx_comp, x[a:b], ctx, cache.state.view(slot, l, "idx_kv"),
                                   cache.state.view(slot, l, "idx_score"), ipool, brow, ps)
                    if E > cfg.index_topk:
                        ik = ipool.view(-1, ipool.shape[-1])[self._entry_slots(brow, 0, E, ratio, ipool.shape[1], ps)].float()
                        sc = (torch.relu(torch.einsum("nhd,ed->nhe", qi[a:b], ik)) * wi[a:b].unsqueeze(-1)).sum(1)
                        sc = sc.masked_fill(~visible, float("-inf"))
                        top = sc.topk(cfg.index_topk, dim=-1)[1]
                        chosen = torch.zeros_like(visible).scatter_(1, top, True)
                        visible = visible & chosen
                keys = torch.cat([keys, ent], 0)
                mask = torch.cat([mask, visible], 1)
            s = torch.einsum("nhd,kd->hnk", q[a:b], keys) * scale
            s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
            sink = lw.sink.view(Hh, 1, 1).expand(Hh, n, 1)
            p = torch.softmax(torch.cat([s, sink], -1), -1)[..., :-1]
            out[a:b] = torch.einsum("hnk,kd->nhd", p, keys)
        return self._project_out(lw, out, meta, compressed)

    def _project_out(self, lw: V4LayerWeights, out, meta: AttnMeta, compressed: bool) -> torch.Tensor:
        """Rotate the rope dims of the attention output back, then the grouped low-rank output projection."""
        cfg = self.cfg
        T, Hh, D = out.shape
        o = self._rotate(out, meta.positions, compressed, inverse=True).to(self.dtype)
        G = cfg.o_groups
        og = o.reshape(T, G, Hh // G * D)
        low = torch.cat([linear(og[:, g].contiguous(), lw.wo_a[g]) for g in range(G)], -1)
        return linear(low, lw.wo_b)

    # ------------------------------------------------------------------ feed-forward
    def _mlp(self, x, w13: Linear, w2: Linear):
        if w13.is_fp8 and x.is_cuda and w13.interleaved:
            return linear(linear(x, w13, silu_mul=True), w2)
        return linear(ref.silu_mul(linear(x, w13)), w2)

    def _moe(self, l: int, lw: V4LayerWeights, x, ids, meta: AttnMeta) -> torch.Tensor:
        cfg = self.cfg
        logits = moe_ops.router_logits(x, lw.router_w)
        if lw.tid2eid is not None:
            idx = lw.tid2eid[ids.long()]
            w = torch.sqrt(F.softplus(logits.float())).gather(1, idx)
            w = w / w.sum(-1, keepdim=True) * cfg.routed_scaling_factor
            idx = idx.to(torch.int32)
        else:
            idx, w = moe_ops.router_topk(logits, lw.router_bias, cfg.num_experts_per_tok, 1, 1, True,
                                         cfg.routed_scaling_factor, "sqrtsoftplus", num_valid=meta.num_valid)
        shared = self._mlp(x, lw.w13, lw.w2)
        if self.comm is not None and self.layout.ep_size > 1:
            routed = self.comm.moe(x, idx, w, lw.experts, cfg.n_routed_experts, num_valid=meta.num_valid)
        else:
            routed = moe_ops.experts_forward(x, idx, w, lw.experts, 0, cfg.n_routed_experts, num_valid=meta.num_valid)
        return routed + shared

    # ------------------------------------------------------------------ forward
    def forward(self, ids: torch.Tensor, meta: AttnMeta, cache) -> torch.Tensor:
        cfg = self.cfg
        h = self.w.embed[ids.long()].unsqueeze(1).expand(-1, cfg.hc_mult, -1).contiguous()          # [T, hc, H]
        for l, lw in enumerate(self.w.layers):
            x, post, comb = self._hc_pre(h, lw.hc_attn)
            a = self._attention(l, lw, self._rms(x, lw.attn_norm), meta, cache)
            h = self._hc_post(a, h, post, comb)
            x, post, comb = self._hc_pre(h, lw.hc_ffn)
            f = self._moe(l, lw, self._rms(x, lw.ffn_norm), ids, meta)
            h = self._hc_post(f, h, post, comb)
        fn, base, scale = self.w.hc_head
        flat = h.reshape(h.shape[0], -1).float()
        rs = torch.rsqrt(flat.square().mean(-1, keepdim=True) + cfg.rms_eps)
        pre = torch.sigmoid((flat @ fn.t()) * rs * scale + base) + cfg.hc_eps
        x = self._rms((pre.unsqueeze(-1) * h.float()).sum(1).to(h.dtype), self.w.final_norm)
        if meta.logit_rows is not None:
            x = x[meta.logit_rows.long()]
        if x.is_cuda and x.dtype == torch.bfloat16 and self.w.lm_head.shape[1] % 64 == 0:
            from ..ops import gemm
            return gemm.bf16_gemm(x.contiguous(), self.w.lm_head, fp32_out=True)
        return (x @ self.w.lm_head.t()).float()

    @staticmethod
    def supports_sequence_parallel(cfg: ModelConfig) -> Optional[str]:
        return "DeepSeek-V4 attention is replicated inside an engine; the fused sequence-parallel layout covers MLA models"
