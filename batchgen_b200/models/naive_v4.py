"""Textbook DeepSeek-V4 oracle: whole-sequence fp32 forward with per-position loops.

No paging, no per-sequence state, no chunking: pooled entries are computed from their definition over absolute
token positions, every query builds its own key set, experts run one token at a time.  It shares only the tensor
source (checkpoint name -> values) with ``models.deepseek_v4``, so a token-for-token match checks that model's
state rings, pending-window bookkeeping, page placement of entries and top-k masking.
(Same role as the readable model the reference vendors next to its DeepSeek-V4 skeleton,
batchgen/models/deepseek/deepseekv4_flash/assets/inference/model.py.)
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import ref
from .weights import WeightSource


class NaiveV4:
    def __init__(self, cfg: ModelConfig, src: WeightSource):
        assert cfg.is_v4
        self.cfg, self.src = cfg, src

    def _g(self, name, shape, kind="normal"):
        return self.src.get(name, shape, kind).float()

    def _rms(self, x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w

    def _rot(self, x, pos: int, compressed: bool, inverse: bool = False):
        """Rotate the last rope dims of a vector (or [heads, D] matrix) for one position."""
        cfg = self.cfg
        rd = cfg.qk_rope_head_dim
        if compressed:
            inv = ref.rope_inv_freq(rd, cfg.compress_rope_theta or cfg.rope_theta, cfg.rope_scaling_factor,
                                    cfg.rope_original_max_pos, cfg.rope_beta_fast, cfg.rope_beta_slow)
        else:
            inv = ref.rope_inv_freq(rd, cfg.rope_theta)
        ang = pos * inv * (-1.0 if inverse else 1.0)
        out = x.clone()
        t = x[..., -rd:]
        even, odd = t[..., 0::2], t[..., 1::2]
        out[..., -rd:][..., 0::2] = even * ang.cos() - odd * ang.sin()
        out[..., -rd:][..., 1::2] = odd * ang.cos() + even * ang.sin()
        return out

    def _entries(self, x, prefix: str, ratio: int, d: int):
        """All pooled entries of the sequence: entry c pools tokens c r .. c r + r - 1 (and, with overlapped
        windows, the r tokens before them through the lower half of the projections)."""
        L, H = x.shape
        c2 = 2 if ratio == 4 else 1
        wkv = self._g(f"{prefix}.wkv.weight", (c2 * d, H))
        wg = self._g(f"{prefix}.wgate.weight", (c2 * d, H))
        ape = self._g(f"{prefix}.ape", (ratio, c2 * d), "bias")
        nw = self._g(f"{prefix}.norm.weight", (d,), "norm")
        out = []
        for c in range(L // ratio):
            rows, gates = [], []
            if c2 == 2 and c > 0:
                for t in range((c - 1) * ratio, c * ratio):
                    rows.append((wkv @ x[t])[:d])
                    gates.append((wg @ x[t] + ape[t % ratio])[:d])
            for t in range(c * ratio, (c + 1) * ratio):
                rows.append((wkv @ x[t])[-d:])
                gates.append((wg @ x[t] + ape[t % ratio])[-d:])
            rows, gates = torch.stack(rows), torch.stack(gates)
            pooled = (rows * torch.softmax(gates, 0)).sum(0)
            out.append(self._rot(self._rms(pooled, nw), c * ratio, True))
        return torch.stack(out) if out else torch.zeros(0, d)

    def _attn(self, x, l: int):
        cfg = self.cfg
        L, H = x.shape
        D, Hh, win, ratio = cfg.head_dim, cfg.num_heads, cfg.sliding_window, cfg.compress_ratios[l]
        a = f"layers.{l}.attn"
        comp = ratio > 0
        qr = self._rms(x @ self._g(f"{a}.wq_a.weight", (cfg.q_lora_rank, H)).t(), self._g(f"{a}.q_norm.weight", (cfg.q_lora_rank,), "norm"))
        q = (qr @ self._g(f"{a}.wq_b.weight", (Hh * D, cfg.q_lora_rank)).t()).view(L, Hh, D)
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        kv = self._rms(x @ self._g(f"{a}.wkv.weight", (D, H)).t(), self._g(f"{a}.kv_norm.weight", (D,), "norm"))
        q = torch.stack([self._rot(q[t], t, comp) for t in range(L)])
        kv = torch.stack([self._rot(kv[t], t, comp) for t in range(L)])
        sink = self._g(f"{a}.attn_sink", (Hh,), "bias")
        ent = self._entries(x, f"{a}.compressor", ratio, D) if comp else None
        if ratio == 4:
            Hi, Di = cfg.index_n_heads, cfg.index_head_dim
            ik = self._entries(x, f"{a}.indexer.compressor", ratio, Di)
            qi = (qr @ self._g(f"{a}.indexer.wq_b.weight", (Hi * Di, cfg.q_lora_rank)).t()).view(L, Hi, Di)
            qi = torch.stack([self._rot(qi[t], t, True) for t in range(L)])
            wi = (x @ self._g(f"{a}.indexer.weights_proj.weight", (Hi, H)).t()) * (Di ** -0.5 * Hi ** -0.5)
        o = torch.zeros(L, Hh, D)
        for t in range(L):
            keys = [kv[p] for p in range(max(0, t - win + 1), t + 1)]
            if comp:
                vis = list(range((t + 1) // ratio))
                if ratio == 4 and len(vis) > cfg.index_topk:
                    sc = torch.stack([(torch.relu(qi[t] @ ik[c]) * wi[t]).sum() for c in vis])
                    vis = sorted(torch.topk(sc, cfg.index_topk)[1].tolist())
                keys += [ent[c] for c in vis]
            K = torch.stack(keys)
            for h in range(Hh):
                s = torch.cat([(K @ q[t, h]) * D ** -0.5, sink[h: h + 1]])
                p = torch.softmax(s, 0)[:-1]
                o[t, h] = p @ K
            o[t] = self._rot(o[t], t, comp, inverse=True)
        G, R = cfg.o_groups, cfg.o_lora_rank
        wo_a = self._g(f"{a}.wo_a.weight", (G * R, Hh * D // G)).view(G, R, -1)
        og = o.reshape(L, G, -1)
        low = torch.cat([og[:, g] @ wo_a[g].t() for g in range(G)], -1)
        return low @ self._g(f"{a}.wo_b.weight", (H, G * R)).t()

    def _expert(self, x, prefix: str, limit: float):
        cfg = self.cfg
        I, H = cfg.moe_intermediate_size, cfg.hidden_size
        gate = x @ self._g(f"{prefix}.w1.weight", (I, H)).t()
        up = x @ self._g(f"{prefix}.w3.weight", (I, H)).t()
        if limit > 0:
            gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        return (F.silu(gate) * up) @ self._g(f"{prefix}.w2.weight", (H, I)).t()

    def _moe(self, x, l: int, ids: List[int]):
        cfg = self.cfg
        E, K, H = cfg.n_routed_experts, cfg.num_experts_per_tok, cfg.hidden_size
        f = f"layers.{l}.ffn"
        scores = torch.sqrt(F.softplus(x @ self._g(f"{f}.gate.weight", (E, H)).t()))
        if l < cfg.num_hash_layers:
            table = self._g(f"{f}.gate.tid2eid", (cfg.vocab_size, E)).topk(K, dim=-1)[1]
            idx = table[torch.tensor(ids)]
        else:
            idx = (scores + self._g(f"{f}.gate.bias", (E,), "bias")).topk(K, dim=-1)[1]
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            w = scores[t, idx[t]]
            w = w / w.sum() * cfg.routed_scaling_factor
            for k in range(K):
                out[t] += w[k] * self._expert(x[t], f"{f}.experts.{int(idx[t, k])}", cfg.swiglu_limit)
        return out + self._expert(x, f"{f}.shared_experts", 0.0)

    def _mix(self, h, prefix: str):
        """Hyper-connection weights of every token: pre [L, hc], post [L, hc], comb [L, hc, hc]."""
        cfg = self.cfg
        hc, H = cfg.hc_mult, cfg.hidden_size
        n = (2 + hc) * hc
        fn, base, scale = (self._g(f"{prefix}_fn", (n, hc * H)), self._g(f"{prefix}_base", (n,), "bias"),
                           self._g(f"{prefix}_scale", (3,), "norm"))
        flat = h.reshape(h.shape[0], -1)
        mixes = (flat @ fn.t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        pre = torch.sigmoid(mixes[:, :hc] * scale[0] + base[:hc]) + cfg.hc_eps
        post = 2 * torch.sigmoid(mixes[:, hc: 2 * hc] * scale[1] + base[hc: 2 * hc])
        comb = torch.softmax(mixes[:, 2 * hc:].view(-1, hc, hc) * scale[2] + base[2 * hc:].view(hc, hc), -1) + cfg.hc_eps
        comb = comb / (comb.sum(1, keepdim=True) + cfg.hc_eps)
        for _ in range(cfg.hc_sinkhorn_iters - 1):
            comb = comb / (comb.sum(2, keepdim=True) + cfg.hc_eps)
            comb = comb / (comb.sum(1, keepdim=True) + cfg.hc_eps)
        return pre, post, comb

    def _block_half(self, h, prefix: str, norm_name: str, fn):
        pre, post, comb = self._mix(h, prefix)
        x = (pre.unsqueeze(-1) * h).sum(1)
        out = fn(self._rms(x, self._g(norm_name, (self.cfg.hidden_size,), "norm")))
        new = torch.zeros_like(h)
        for j in range(self.cfg.hc_mult):
            new[:, j] = post[:, j: j + 1] * out + sum(comb[:, i, j: j + 1] * h[:, i] for i in range(self.cfg.hc_mult))
        return new

    @torch.no_grad()
    def logits(self, ids: List[int]) -> torch.Tensor:
        cfg = self.cfg
        H, hc = cfg.hidden_size, cfg.hc_mult
        emb = self._g("embed.weight", (cfg.vocab_size, H))[torch.tensor(ids)]
        h = emb.unsqueeze(1).repeat(1, hc, 1)
        for l in range(cfg.num_layers):
            p = f"layers.{l}"
            h = self._block_half(h, f"{p}.hc_attn", f"{p}.attn_norm.weight", lambda x: self._attn(x, l))
            h = self._block_half(h, f"{p}.hc_ffn", f"{p}.ffn_norm.weight", lambda x: self._moe(x, l, ids))
        fn, base, scale = self._g("hc_head_fn", (hc, hc * H)), self._g("hc_head_base", (hc,), "bias"), self._g("hc_head_scale", (1,), "norm")
        flat = h.reshape(h.shape[0], -1)
        pre = torch.sigmoid((flat @ fn.t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * scale + base) + cfg.hc_eps
        x = self._rms((pre.unsqueeze(-1) * h).sum(1), self._g("norm.weight", (H,), "norm"))
        return x @ self._g("head.weight", (cfg.vocab_size, H)).t()

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(max_new_tokens):
            nxt = int(self.logits(ids)[-1].argmax())
            out.append(nxt)
            ids.append(nxt)
        return out
