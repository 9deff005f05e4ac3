"""Naive oracle: the same architecture written the textbook way.

No paging, no KV cache, no absorption, no fusion, no parallelism: every call recomputes the whole
sequence in fp32 with *expanded* MLA keys/values (k_nope = W_UK c_kv, v = W_UV c_kv) and a per-token
Python loop over experts.  It shares only the checkpoint-name -> tensor source with the engine, so a
token-for-token match between the two checks the engine's paging, absorption, routing, dispatch and
scheduling logic.  (Same role as the reference's readable torch backend,
batchgen/attention/mla/torch_backend.py, and its HF-oracle test harness tests/kimi_k3_harness.py.)
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import ref
from .weights import WeightSource


class NaiveModel:
    def __init__(self, cfg: ModelConfig, src: WeightSource):
        self.cfg, self.src = cfg, src

    def _g(self, name, shape, kind="normal"):
        return self.src.get(name, shape, kind).float()

    def _rms(self, x, name, n):
        w = self._g(name, (n,), "norm")
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w

    def _rope(self, x, positions):
        cfg = self.cfg
        inv = ref.rope_inv_freq(cfg.qk_rope_head_dim if cfg.is_mla else cfg.head_dim, cfg.rope_theta, cfg.rope_scaling_factor,
                                cfg.rope_original_max_pos, cfg.rope_beta_fast, cfg.rope_beta_slow)
        cos, sin = ref.rope_cos_sin(positions, inv)
        return ref.apply_rope(x, cos, sin, cfg.rope_interleaved)

    def _mlp(self, x, prefix, inter, hid):
        g = self._g(f"{prefix}.gate_proj.weight", (inter, hid))
        u = self._g(f"{prefix}.up_proj.weight", (inter, hid))
        d = self._g(f"{prefix}.down_proj.weight", (hid, inter))
        gate, up = x @ g.t(), x @ u.t()
        if self.cfg.activation == "swiglu_clamped":       # GPT-OSS: clamp, (up + 1) * gate * sigmoid(1.702 gate)
            gate, up = gate.clamp(max=7.0), up.clamp(-7.0, 7.0)
            return ((up + 1.0) * gate * torch.sigmoid(1.702 * gate)) @ d.t()
        return (F.silu(gate) * up) @ d.t()

    def _gqa(self, x, l, p, pos):
        """Grouped-query attention over the whole sequence: every query head reads the key/value head of its group."""
        cfg = self.cfg
        L, H, D, Hq, Hkv = x.shape[0], cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        a = f"{p}.self_attn"

        def proj(name, heads):
            y = x @ self._g(f"{a}.{name}_proj.weight", (heads * D, H)).t()
            if cfg.attention_bias:
                y = y + self._g(f"{a}.{name}_proj.bias", (heads * D,), "bias")
            return y.view(L, heads, D)

        q, k, v = self._rope(proj("q", Hq), pos), self._rope(proj("k", Hkv), pos), proj("v", Hkv)
        out = torch.zeros(L, Hq, D)
        window = cfg.sliding_window if (cfg.sliding_window and l % 2 == 0) else 0
        sinks = self._g(f"{a}.sinks", (Hq,), "bias") if cfg.attention_sinks else None
        for h in range(Hq):
            kh, vh = k[:, h // (Hq // Hkv)], v[:, h // (Hq // Hkv)]
            for t in range(L):
                first = max(0, t + 1 - window) if window else 0
                sc = (kh[first: t + 1] @ q[t, h]) * cfg.softmax_scale
                if sinks is not None:
                    sc = torch.cat([sc, sinks[h: h + 1]])
                pr = torch.softmax(sc, 0)[: t + 1 - first]
                out[t, h] = pr @ vh[first: t + 1]
        return out.reshape(L, Hq * D) @ self._g(f"{a}.o_proj.weight", (H, Hq * D)).t()

    @torch.no_grad()
    def logits(self, ids: List[int]) -> torch.Tensor:
        """Full-sequence forward -> fp32 logits [len(ids), vocab]."""
        cfg = self.cfg
        H, L = cfg.hidden_size, len(ids)
        pos = torch.arange(L)
        h = self._g("model.embed_tokens.weight", (cfg.vocab_size, H))[torch.tensor(ids)]
        for l in range(cfg.num_layers):
            p = f"model.layers.{l}"
            x = self._rms(h, f"{p}.input_layernorm.weight", H)
            if cfg.layer_is_kda(l) or not cfg.is_mla:
                h = h + (self._kda(x, p) if cfg.layer_is_kda(l) else self._gqa(x, l, p, pos))
                x = self._rms(h, f"{p}.post_attention_layernorm.weight", H)
                h = h + (self._moe(x, p) if cfg.is_moe_layer(l) else self._mlp(x, f"{p}.mlp", cfg.intermediate_size, H))
                continue
            # ---- MLA, expanded form
            q_a = x @ self._g(f"{p}.self_attn.q_a_proj.weight", (cfg.q_lora_rank, H)).t()
            q_a = self._rms(q_a, f"{p}.self_attn.q_a_layernorm.weight", cfg.q_lora_rank)
            q = (q_a @ self._g(f"{p}.self_attn.q_b_proj.weight",
                               (cfg.num_heads * cfg.qk_head_dim, cfg.q_lora_rank)).t()).view(L, cfg.num_heads, -1)
            q_nope, q_pe = q[..., : cfg.qk_nope_head_dim], self._rope(q[..., cfg.qk_nope_head_dim:], pos)
            kv_a = x @ self._g(f"{p}.self_attn.kv_a_proj_with_mqa.weight",
                               (cfg.kv_lora_rank + cfg.qk_rope_head_dim, H)).t()
            c_kv = self._rms(kv_a[:, : cfg.kv_lora_rank], f"{p}.self_attn.kv_a_layernorm.weight", cfg.kv_lora_rank)
            k_pe = self._rope(kv_a[:, cfg.kv_lora_rank:], pos)
            kvb = self._g(f"{p}.self_attn.kv_b_proj.weight",
                          (cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank))
            kv = (c_kv @ kvb.t()).view(L, cfg.num_heads, cfg.qk_nope_head_dim + cfg.v_head_dim)
            k_nope, v = kv[..., : cfg.qk_nope_head_dim], kv[..., cfg.qk_nope_head_dim:]
            s = (torch.einsum("qhd,khd->hqk", q_nope, k_nope) + torch.einsum("qhd,kd->hqk", q_pe, k_pe))
            s = s * cfg.softmax_scale
            causal = torch.ones(L, L, dtype=torch.bool).tril()
            if cfg.has_dsa:
                keep = self._dsa_mask(l, p, x, q_a, pos)          # [L, L] bool
                causal = causal & keep
            s = s.masked_fill(~causal.unsqueeze(0), float("-inf"))
            o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(L, -1)
            h = h + o @ self._g(f"{p}.self_attn.o_proj.weight", (H, cfg.num_heads * cfg.v_head_dim)).t()
            # ---- feed-forward
            x = self._rms(h, f"{p}.post_attention_layernorm.weight", H)
            if cfg.is_moe_layer(l):
                h = h + self._moe(x, p)
            else:
                h = h + self._mlp(x, f"{p}.mlp", cfg.intermediate_size, H)
        h = self._rms(h, "model.norm.weight", H)
        head = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
        return h @ self._g(head, (cfg.vocab_size, H)).t()

    def _kda(self, x, p):
        """Gated delta-rule linear attention over the whole sequence, one token at a time."""
        cfg = self.cfg
        Hk, D, r, H, L = cfg.kda_num_heads, cfg.kda_head_dim, cfg.kda_rank, cfg.hidden_size, x.shape[0]
        a = f"{p}.self_attn"

        def conv(name):
            raw = x @ self._g(f"{a}.{name}_proj.weight", (Hk * D, H)).t()
            w = self._g(f"{a}.{name}_conv1d.weight", (Hk * D, 4), "bias")
            padded = torch.cat([torch.zeros(3, Hk * D), raw], 0)
            y = sum(padded[i:i + L] * w[:, i] for i in range(4))
            return F.silu(y).view(L, Hk, D)

        q, k, v = conv("q"), conv("k"), conv("v")
        q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        f = (x @ self._g(f"{a}.f_a_proj.weight", (r, H)).t()) @ self._g(f"{a}.f_b_proj.weight", (Hk * D, r)).t()
        A = self._g(f"{a}.A_log", (Hk,), "bias").exp()
        decay = torch.exp(-A.view(1, Hk, 1) * F.softplus(f.view(L, Hk, D) + self._g(f"{a}.dt_bias", (Hk * D,), "bias").view(1, Hk, D)))
        beta = torch.sigmoid(x @ self._g(f"{a}.b_proj.weight", (Hk, H)).t())
        z = (x @ self._g(f"{a}.g_proj.weight", (Hk * D, H)).t()).view(L, Hk, D)
        S = torch.zeros(Hk, D, D)
        o = torch.zeros(L, Hk, D)
        for t in range(L):
            S = S * decay[t].unsqueeze(-1)
            pred = (S * k[t].unsqueeze(-1)).sum(1)
            S = S + k[t].unsqueeze(-1) * (beta[t].unsqueeze(-1) * (v[t] - pred)).unsqueeze(1)
            o[t] = (S * q[t].unsqueeze(-1)).sum(1)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * self._g(f"{a}.o_norm.weight", (D,), "norm")
        o = (o * torch.sigmoid(z)).reshape(L, Hk * D)
        return o @ self._g(f"{a}.o_proj.weight", (H, Hk * D)).t()

    def _moe(self, x, p):
        cfg = self.cfg
        E, I, eh, H = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.expert_hidden, cfg.hidden_size
        logits = x @ self._g(f"{p}.mlp.gate.weight", (E, H)).t()
        bias = (self._g(f"{p}.mlp.gate.e_score_correction_bias", (E,), "bias")
                if cfg.scoring_func in ("sigmoid", "sqrtsoftplus") else None)
        idx, w = ref.router_topk(logits, bias, cfg.num_experts_per_tok, cfg.n_group, cfg.topk_group,
                                 cfg.norm_topk_prob, cfg.routed_scaling_factor, cfg.scoring_func)
        xin = x
        if cfg.moe_latent_size:
            xin = x @ self._g(f"{p}.mlp.latent_down_proj.weight", (eh, H)).t()
        out = torch.zeros(x.shape[0], eh)
        for t in range(x.shape[0]):
            for k in range(cfg.num_experts_per_tok):
                e = int(idx[t, k])
                out[t] += w[t, k] * self._mlp(xin[t: t + 1], f"{p}.mlp.experts.{e}", I, eh)[0]
        if cfg.moe_latent_size:
            out = self._rms(out, f"{p}.mlp.latent_norm.weight", eh)
            out = out @ self._g(f"{p}.mlp.latent_up_proj.weight", (H, eh)).t()
        if cfg.n_shared_experts:
            shared = self._mlp(x, f"{p}.mlp.shared_experts", I * cfg.n_shared_experts, H)
            if cfg.shared_expert_gate:
                shared = shared * torch.sigmoid(x @ self._g(f"{p}.mlp.shared_expert_gate.weight", (1, H)).t())
            out = out + shared
        return out

    def _dsa_mask(self, l, p, x, q_a_normed, pos):
        """Per-query key mask from the lightning indexer (index keys pass through e4m3, as cached)."""
        cfg = self.cfg
        L = x.shape[0]
        if not cfg.layer_has_indexer(l):
            src_layer = max(i for i in cfg.indexer_full_layers if i <= l)
            return self._dsa_cache[src_layer]
        Hi, Di, rd, H = cfg.index_n_heads, cfg.index_head_dim, cfg.qk_rope_head_dim, cfg.hidden_size
        ip = f"{p}.self_attn.indexer"
        k = x @ self._g(f"{ip}.wk.weight", (Di, H)).t()
        k = F.layer_norm(k, (Di,), self._g(f"{ip}.k_norm.weight", (Di,), "norm"),
                         self._g(f"{ip}.k_norm.bias", (Di,), "bias"), 1e-6)
        k = torch.cat([self._rope(k[:, :rd], pos), k[:, rd:]], -1)
        kq, ks = ref.index_k_quant(k)
        q = (q_a_normed @ self._g(f"{ip}.wq_b.weight", (Hi * Di, cfg.q_lora_rank)).t()).view(L, Hi, Di)
        q = torch.cat([self._rope(q[..., :rd], pos), q[..., rd:]], -1)
        gates = (x @ self._g(f"{ip}.weights_proj.weight", (Hi, H)).t()) * (Hi ** -0.5) * (Di ** -0.5)
        keep = torch.zeros(L, L, dtype=torch.bool)
        for t in range(L):
            n = t + 1
            if n <= cfg.index_topk:
                keep[t, :n] = True
            else:
                sc = ref.indexer_scores(q[t], gates[t], kq[:n], ks[:n])
                keep[t, torch.topk(sc, cfg.index_topk)[1]] = True
        if not hasattr(self, "_dsa_cache"):
            self._dsa_cache = {}
        self._dsa_cache[l] = keep
        return keep

    @torch.no_grad()
    def generate(self, prompt: List[int], max_new_tokens: int) -> List[int]:
        ids = list(prompt)
        out = []
        for _ in range(max_new_tokens):
            nxt = int(self.logits(ids)[-1].argmax())
            out.append(nxt)
            ids.append(nxt)
        return out
