"""Plain-PyTorch reference implementations of every hot operator.

These run on any device, compute in fp32, and are (a) the CPU execution path of the engine
(the tiny fp32 correctness configuration) and (b) the numerics oracle each CUDA kernel is
tested against.  They favour clarity over speed.

Reference parity (behaviour, not code): FP8 block quantisation follows
``batchgen/quantization/block_quantization.py`` and ``batchgen_kernels/triton/fp8_quantize.py:8-80``
(1x128 activation scales = amax/448, 128x128 weight scales); the MLA math follows
``batchgen/attention/mla/torch_backend.py:9-194``; the router follows
``batchgen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:793-846``; the MXFP4 decode
follows ``batchgen/quantization/mxfp4.py:30``; the DSA indexer follows
``batchgen/models/glm/glm5/model.py:610-700``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


# --------------------------------------------------------------------------- quantisation
def _ceil_pow2(x: torch.Tensor) -> torch.Tensor:
    """Round positive fp32 values up to the next power of two (UE8M0-representable)."""
    return torch.exp2(torch.ceil(torch.log2(x.clamp_min(1e-30))))


def act_quant(x: torch.Tensor, block: int = 128, pow2_scale: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-``block`` e4m3 quantisation.  x: [T, K] -> (q [T, K] e4m3, s [T, K/block] fp32).

    scale = max(amax, 1e-4) / 448; q = x * (1/scale) rounded to nearest e4m3 (saturating)."""
    T, K = x.shape
    assert K % block == 0, (K, block)
    xf = x.float().view(T, K // block, block)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-4)
    s = amax / FP8_MAX
    if pow2_scale:
        s = _ceil_pow2(s)
    q = (xf * (1.0 / s).unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(T, K), s


def weight_quant_block(w: torch.Tensor, block: int = 128, pow2_scale: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128 block e4m3 quantisation of a weight [N, K] -> (q [N, K], s [ceil(N/b), ceil(K/b)])."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    wv = wp.view(nb, block, kb, block)
    amax = wv.abs().amax(dim=(1, 3)).clamp_min(1e-4)
    s = amax / FP8_MAX
    if pow2_scale:
        s = _ceil_pow2(s)
    q = (wv / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(nb * block, kb * block)[:N, :K].contiguous(), s


def dequant_block(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    se = s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * se


def dequant_act(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    return q.float() * s.repeat_interleave(block, 1)[:, : q.shape[1]]


def fp8_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
             out_dtype: torch.dtype = torch.float32, block: int = 128) -> torch.Tensor:
    """out[T, N] = (xq * xs) @ (wq * ws)^T with fp32 accumulation."""
    return (dequant_act(xq, xs, block) @ dequant_block(wq, ws, block).t()).to(out_dtype)


def grouped_fp8_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor,
                     offsets: torch.Tensor, out_dtype: torch.dtype = torch.float32,
                     block: int = 128) -> torch.Tensor:
    """Ragged grouped GEMM.  Rows ``offsets[e]:offsets[e+1]`` of x use expert e.
    wq: [E, N, K], ws: [E, N/b, K/b], offsets: [E+1] (int)."""
    E, N, _ = wq.shape
    out = torch.zeros(xq.shape[0], N, dtype=out_dtype, device=xq.device)
    off = offsets.tolist()
    for e in range(E):
        a, b = off[e], off[e + 1]
        if b > a:
            out[a:b] = fp8_gemm(xq[a:b], xs[a:b], wq[e], ws[e], out_dtype, block)
    return out


# --------------------------------------------------------------------------- MXFP4
_E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _e2m1_lut(device) -> torch.Tensor:
    v = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=device)
    return torch.cat([v, -v])


def mxfp4_quant(w: torch.Tensor, block: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise [N, K] to MXFP4: packed e2m1 nibbles [N, K/2] uint8 (low nibble = even k)
    plus e8m0 scales [N, K/block] uint8 (value = 2^(s-127))."""
    N, K = w.shape
    assert K % block == 0
    wf = w.float().view(N, K // block, block)
    amax = wf.abs().amax(-1).clamp_min(2.0 ** -126)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scale = torch.exp2(exp)
    x = wf / scale.unsqueeze(-1)
    lut = torch.tensor(_E2M1_VALUES, dtype=torch.float32, device=w.device)
    mag = x.abs().unsqueeze(-1)
    code = (mag - lut).abs().argmin(-1)
    code = code + (x < 0).long() * 8
    code = code.view(N, K)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).to(torch.uint8)
    return packed, (exp + 127).to(torch.uint8)


def mxfp4_dequant(packed: torch.Tensor, scales: torch.Tensor, block: int = 32) -> torch.Tensor:
    N, Kh = packed.shape
    lut = _e2m1_lut(packed.device)
    lo = lut[(packed & 0xF).long()]
    hi = lut[(packed >> 4).long()]
    w = torch.stack([lo, hi], dim=-1).view(N, Kh * 2)
    s = torch.exp2(scales.float() - 127.0).repeat_interleave(block, 1)
    return w * s


# --------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], w: torch.Tensor,
                eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """residual' = x + residual (kept in x.dtype); y = rmsnorm(residual')."""
    r = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(r, w, eps), r


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


# --------------------------------------------------------------------------- rope
def _yarn_find_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def rope_inv_freq(dim: int, theta: float, scaling_factor: float = 1.0, original_max_pos: int = 4096,
                  beta_fast: float = 32.0, beta_slow: float = 1.0) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if scaling_factor <= 1.0:
        return inv
    low = max(math.floor(_yarn_find_dim(beta_fast, dim, theta, original_max_pos)), 0)
    high = min(math.ceil(_yarn_find_dim(beta_slow, dim, theta, original_max_pos)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    return inv / scaling_factor * (1 - mask) + inv * mask


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, mscale: float = 1.0):
    ang = positions.float().unsqueeze(-1) * inv_freq.to(positions.device)
    return ang.cos() * mscale, ang.sin() * mscale


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = True) -> torch.Tensor:
    """x: [T, ..., D]; cos/sin: [T, D/2].  interleaved pairs (2i, 2i+1) or half-split (i, i+D/2)."""
    shape = x.shape
    D = shape[-1]
    xf = x.float()
    while cos.dim() < xf.dim():
        cos = cos.unsqueeze(1)
        sin = sin.unsqueeze(1)
    if interleaved:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        o1 = x1 * cos - x2 * sin
        o2 = x2 * cos + x1 * sin
        out = torch.stack([o1, o2], dim=-1).view(shape)
    else:
        x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- router
def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int = 1,
                topk_group: int = 1, norm_topk_prob: bool = True, scale: float = 1.0,
                scoring: str = "sigmoid") -> Tuple[torch.Tensor, torch.Tensor]:
    """logits: [T, E] fp32 -> (idx [T, k] int32 sorted by descending choice score, w [T, k] fp32).

    sigmoid scoring (DeepSeek-V3, GLM, Kimi): choice = sigmoid(logit) + bias; group-limited selection keeps
    the ``topk_group`` groups with the largest (sum of top-2 choice scores); weights come from the
    *unbiased* sigmoid, normalised and multiplied by ``scale``.
    softmax scoring (GPT-OSS, Mixtral): top-k on logits, softmax over the selected logits.
    softmax_all scoring (DeepSeek-V2, Qwen2-MoE): softmax over every expert first; group-limited selection
    ranks groups by their best expert; the weights are the selected probabilities, renormalised only when
    ``norm_topk_prob`` is set.
    sqrtsoftplus scoring (DeepSeek-V4): score = sqrt(softplus(logit)), chosen with the bias added, weights
    from the unbiased score."""
    T, E = logits.shape
    lf = logits.float()
    if scoring == "softmax":
        val, idx = torch.topk(lf, top_k, dim=-1)
        return idx.to(torch.int32), torch.softmax(val, dim=-1) * scale
    if scoring == "sigmoid":
        scores = torch.sigmoid(lf)
    elif scoring == "softmax_all":
        scores = torch.softmax(lf, dim=-1)
    elif scoring == "sqrtsoftplus":
        scores = torch.sqrt(torch.nn.functional.softplus(lf))
    else:
        raise ValueError(f"unknown router scoring {scoring!r}")
    choice = scores if bias is None else scores + bias.float().unsqueeze(0)
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        gscore = g.max(-1)[0] if scoring == "softmax_all" else g.topk(2, dim=-1)[0].sum(-1)
        gidx = gscore.topk(topk_group, dim=-1)[1]
        gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
        emask = gmask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
        choice = choice.masked_fill(emask == 0, float("-inf"))
    _, idx = torch.topk(choice, top_k, dim=-1)
    w = scores.gather(1, idx)
    if top_k > 1 and norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), w * scale


# --------------------------------------------------------------------------- MoE plumbing
def moe_permute(topk_idx: torch.Tensor, num_experts: int, expert_lo: int = 0,
                expert_hi: Optional[int] = None, align: int = 1):
    """Group the (token, k) pairs routed to experts [lo, hi) by expert.

    Returns (src_row [R] int64: token of each grouped row, -1 for alignment padding,
             pos [T, k] int64: grouped row of each pair or -1 if not local,
             offsets [E_local + 1] int64 with every segment start aligned to ``align``)."""
    expert_hi = num_experts if expert_hi is None else expert_hi
    T, K = topk_idx.shape
    flat = topk_idx.reshape(-1).long()
    local = (flat >= expert_lo) & (flat < expert_hi)
    el = expert_hi - expert_lo
    counts = torch.bincount((flat[local] - expert_lo), minlength=el)
    padded = ((counts + align - 1) // align) * align
    offsets = torch.zeros(el + 1, dtype=torch.int64, device=topk_idx.device)
    offsets[1:] = torch.cumsum(padded, 0)
    R = int(offsets[-1].item())
    src_row = torch.full((R,), -1, dtype=torch.int64, device=topk_idx.device)
    pos = torch.full((T * K,), -1, dtype=torch.int64, device=topk_idx.device)
    pair_ids = torch.nonzero(local, as_tuple=False).squeeze(-1)
    if pair_ids.numel():
        e = flat[pair_ids] - expert_lo
        order = torch.argsort(e, stable=True)
        pair_sorted = pair_ids[order]
        e_sorted = e[order]
        starts = torch.cumsum(counts, 0) - counts
        rank_in_e = torch.arange(pair_sorted.numel(), device=topk_idx.device) - starts[e_sorted]
        rows = offsets[e_sorted] + rank_in_e
        src_row[rows] = pair_sorted // K
        pos[pair_sorted] = rows
    return src_row, pos.view(T, K), offsets


def moe_combine(expert_out: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out[t] = sum_k w[t,k] * expert_out[pos[t,k]] in k order (fp32 accumulation); pos<0 skipped."""
    T, K = pos.shape
    H = expert_out.shape[-1]
    acc = torch.zeros(T, H, dtype=torch.float32, device=expert_out.device)
    if expert_out.shape[0] == 0:            # none of this rank's experts was chosen in this step
        return acc.to(out_dtype or expert_out.dtype)
    for k in range(K):
        p = pos[:, k]
        valid = p >= 0
        rows = expert_out[p.clamp_min(0)].float() * weights[:, k].float().unsqueeze(-1)
        acc += torch.where(valid.unsqueeze(-1), rows, torch.zeros_like(rows))
    return acc.to(out_dtype or expert_out.dtype)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up: [T, 2I] with gate in the first half -> silu(gate) * up."""
    I = gate_up.shape[-1] // 2
    g, u = gate_up[..., :I].float(), gate_up[..., I:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def swiglu_clamped(gate_up: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """GPT-OSS activation: gate clamped above, up clamped both sides, (up + 1) * gate*sigmoid(alpha*gate)."""
    I = gate_up.shape[-1] // 2
    g = gate_up[..., :I].float().clamp(max=limit)
    u = gate_up[..., I:].float().clamp(-limit, limit)
    return ((u + 1.0) * g * torch.sigmoid(alpha * g)).to(gate_up.dtype)


# --------------------------------------------------------------------------- paged KV + MLA
def kv_cache_write(cache: torch.Tensor, rows: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """cache: [P, page, D]; rows: [T, D]; slot_mapping: [T] flat slot (page*page_size+offset), -1 = skip."""
    P, S, D = cache.shape
    valid = slot_mapping >= 0
    flat = cache.view(P * S, D)
    flat[slot_mapping[valid].long()] = rows[valid].to(cache.dtype)


def mla_kv_prepare(kv_a: torch.Tensor, norm_w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   kv_lora: int, eps: float, interleaved: bool) -> torch.Tensor:
    """kv_a: [T, kv_lora + rope] -> cache row [T, kv_lora + rope] = [rmsnorm(c_kv) | rope(k_pe)]."""
    c = rmsnorm(kv_a[:, :kv_lora], norm_w, eps)
    k_pe = apply_rope(kv_a[:, kv_lora:], cos, sin, interleaved)
    return torch.cat([c, k_pe], dim=-1)


def gather_paged(cache: torch.Tensor, block_table_row: torch.Tensor, length: int) -> torch.Tensor:
    """Rows 0..length-1 of one sequence from cache [P, page, D] via its block table -> [length, D]."""
    P, S, D = cache.shape
    n_pages = (length + S - 1) // S
    pages = cache[block_table_row[:n_pages].long()]
    return pages.reshape(n_pages * S, D)[:length]


def mla_decode(q_abs: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
               seqlens: torch.Tensor, scale: float, kv_lora: int) -> torch.Tensor:
    """Absorbed MLA decode.  q_abs: [B, H, kv_lora], q_pe: [B, H, rope], cache [P, page, kv_lora+rope].
    Returns the latent-space output [B, H, kv_lora] (fp32 math, cast to q dtype)."""
    B, H, _ = q_abs.shape
    out = torch.zeros(B, H, kv_lora, dtype=torch.float32, device=q_abs.device)
    for b in range(B):
        L = int(seqlens[b])
        if L <= 0:
            continue
        kv = gather_paged(cache, block_table[b], L).float()
        c, kpe = kv[:, :kv_lora], kv[:, kv_lora:]
        s = (q_abs[b].float() @ c.t() + q_pe[b].float() @ kpe.t()) * scale
        out[b] = torch.softmax(s, dim=-1) @ c
    return out.to(q_abs.dtype)


def mla_prefill(q_abs: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                cu_seqlens: Sequence[int], ctx_lens: Sequence[int], scale: float, kv_lora: int) -> torch.Tensor:
    """Varlen causal absorbed MLA over the paged cache (the new tokens' KV must already be
    written).  Sequence i owns query rows cu_seqlens[i]:cu_seqlens[i+1]; ``ctx_lens[i]`` is the
    number of tokens already cached *before* those rows (prefix-hit / chunked prefill), so query
    j attends to cache positions 0..ctx+j."""
    T, H, _ = q_abs.shape
    out = torch.zeros(T, H, kv_lora, dtype=torch.float32, device=q_abs.device)
    for i in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        n = b - a
        if n == 0:
            continue
        ctx = int(ctx_lens[i])
        kv = gather_paged(cache, block_table[i], ctx + n).float()
        c, kpe = kv[:, :kv_lora], kv[:, kv_lora:]
        s = (torch.einsum("nhd,ld->hnl", q_abs[a:b].float(), c)
             + torch.einsum("nhd,ld->hnl", q_pe[a:b].float(), kpe)) * scale
        qpos = torch.arange(n, device=s.device).unsqueeze(-1) + ctx
        kpos = torch.arange(ctx + n, device=s.device).unsqueeze(0)
        s = s.masked_fill((kpos > qpos).unsqueeze(0), float("-inf"))
        out[a:b] = torch.einsum("hnl,ld->nhd", torch.softmax(s, dim=-1), c)
    return out.to(q_abs.dtype)


def sparse_mla_decode(q_abs, q_pe, cache, block_table, sel_idx, sel_len, scale, kv_lora):
    """MLA decode over selected token positions only.  sel_idx: [B, topk] logical positions
    (first sel_len[b] valid)."""
    B, H, _ = q_abs.shape
    P, S, D = cache.shape
    out = torch.zeros(B, H, kv_lora, dtype=torch.float32, device=q_abs.device)
    for b in range(B):
        n = int(sel_len[b])
        if n <= 0:
            continue
        posn = sel_idx[b, :n].long()
        slots = block_table[b][posn // S].long() * S + posn % S
        kv = cache.view(P * S, D)[slots].float()
        c, kpe = kv[:, :kv_lora], kv[:, kv_lora:]
        s = (q_abs[b].float() @ c.t() + q_pe[b].float() @ kpe.t()) * scale
        out[b] = torch.softmax(s, dim=-1) @ c
    return out.to(q_abs.dtype)


# --------------------------------------------------------------------------- GQA
def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, q_start: int = 0,
                  window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal GQA for one sequence.  q: [n, Hq, D]; k, v: [L, Hkv, D]; query j sits at absolute
    position q_start + j.  ``window`` > 0 restricts keys to the last ``window`` positions;
    ``sinks`` [Hq] adds a per-head logit to the softmax denominator only."""
    n, Hq, D = q.shape
    L, Hkv, _ = k.shape
    rep = Hq // Hkv
    kf = k.float().repeat_interleave(rep, 1)
    vf = v.float().repeat_interleave(rep, 1)
    s = torch.einsum("nhd,lhd->hnl", q.float(), kf) * scale
    qpos = torch.arange(n, device=q.device).unsqueeze(-1) + q_start
    kpos = torch.arange(L, device=q.device).unsqueeze(0)
    mask = kpos > qpos
    if window > 0:
        mask = mask | (kpos <= qpos - window)
    s = s.masked_fill(mask.unsqueeze(0), float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(Hq, 1, 1).expand(Hq, n, 1)
        p = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :L]
    else:
        p = torch.softmax(s, dim=-1)
    return torch.einsum("hnl,lhd->nhd", p, vf).to(q.dtype)


# --------------------------------------------------------------------------- DSA indexer
def index_k_quant(k: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Index keys [T, D] -> (e4m3 [T, D], fp32 scale [T]); scale = max(amax, 1e-4) / 448, applied
    as a reciprocal multiply."""
    amax = k.float().abs().amax(-1).clamp_min(1e-4)
    s = amax / FP8_MAX
    q = (k.float() * (1.0 / s).unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q, s


def indexer_scores(q: torch.Tensor, head_w: torch.Tensor, kq: torch.Tensor, ks: torch.Tensor) -> torch.Tensor:
    """score[t] = sum_h head_w[h] * relu(q[h] . k[t]) for one query.  q: [Hi, D], kq: [L, D] e4m3,
    ks: [L] -> [L] fp32."""
    k = kq.float() * ks.float().unsqueeze(-1)
    return (torch.relu(q.float() @ k.t()) * head_w.float().unsqueeze(-1)).sum(0)


def topk_select(scores: torch.Tensor, length: int, k: int) -> Tuple[torch.Tensor, int]:
    """Indices of the k largest of scores[:length] (all of them if length <= k)."""
    if length <= k:
        return torch.arange(length, device=scores.device, dtype=torch.int32), length
    return torch.topk(scores[:length], k)[1].to(torch.int32), k


# --------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           generator: Optional[torch.Generator] = None, uniform: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row temperature / top-k / top-p sampling.  temperature <= 0 means greedy.
    ``uniform`` ([T] in [0,1)) makes the draw deterministic for kernel parity tests."""
    T, V = logits.shape
    lf = logits.float()
    greedy = lf.argmax(-1)
    temp = temperature.float().clamp_min(1e-6).unsqueeze(-1)
    probs = torch.softmax(lf / temp, dim=-1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    ranks = torch.arange(V, device=logits.device).unsqueeze(0)
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V)).unsqueeze(-1)
    keep = ranks < k
    # the filters are sequential (batchgen/sampling.py:417-461): the nucleus is taken on the distribution
    # renormalised over the top-k survivors; a token stays while the mass before it is at most top_p
    sk = torch.where(keep, sp, torch.zeros_like(sp))
    zk = sk.sum(-1, keepdim=True)
    cum = torch.cumsum(sk, -1)
    tp = top_p.float().unsqueeze(-1)
    keep &= ((cum - sk) <= tp * zk) | (tp >= 1.0)
    keep[:, 0] = True
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    sp = sp / sp.sum(-1, keepdim=True)
    if uniform is None:
        uniform = torch.rand(T, device=logits.device, generator=generator)
    c = torch.cumsum(sp, -1)
    choice = (c < uniform.unsqueeze(-1) * c[:, -1:]).sum(-1).clamp_max(V - 1)
    sampled = si.gather(1, choice.unsqueeze(-1)).squeeze(-1)
    return torch.where(temperature <= 0, greedy, sampled)
