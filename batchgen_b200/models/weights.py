"""Weight containers, random initialisation and sharding.

Tensors are created per *checkpoint name* (HF DeepSeek-V3 naming, which the converter's module
keys ``attn_L`` / ``shared_expert_L`` / ``routed_expert_L_E`` also use —
batchgen/models/deepseek/deepseekv3/Parallel_Strategy_Manager.py:225-290) from a generator seeded
by ``hash(seed, name)``, so every rank of a TP/EP layout derives bit-identical full tensors and
cuts its own shard, and the naive oracle can rebuild exactly the same model.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..ops import ref
from ..ops.moe import ExpertWeights

FP8 = torch.float8_e4m3fn


@dataclass
class ParallelLayout:
    """Which slice of the model one rank owns."""
    tp_rank: int = 0
    tp_size: int = 1     # attention heads / dense-MLP / shared-expert / vocab sharding
    ep_rank: int = 0
    ep_size: int = 1     # routed experts sharding (contiguous blocks)
    sequence_parallel: bool = False   # row-sharded residual stream: shared experts and lm_head replicated

    def expert_range(self, n_experts: int) -> Tuple[int, int]:
        per = n_experts // self.ep_size
        return self.ep_rank * per, (self.ep_rank + 1) * per

    def head_range(self, n_heads: int) -> Tuple[int, int]:
        per = n_heads // self.tp_size
        return self.tp_rank * per, (self.tp_rank + 1) * per


@dataclass
class Linear:
    """A linear weight [N, K]; ``s`` holds 128x128 block scales when ``w`` is e4m3."""
    w: torch.Tensor
    s: Optional[torch.Tensor] = None
    interleaved: bool = False   # gate/up rows in the tile-interleaved order of the fused SiLU epilogue

    @property
    def is_fp8(self) -> bool:
        return self.s is not None

    def interleave_gate_up_(self) -> "Linear":
        """GPU fp8 gate|up weights: reorder rows so the GEMM epilogue can fuse SiLU(gate)*up."""
        if self.is_fp8 and self.w.is_cuda and not self.interleaved and (self.w.shape[0] // 2) % 128 == 0:
            from ..ops.gemm import interleave_gate_up_rows
            perm = interleave_gate_up_rows(self.w.shape[0], self.w.device)
            self.w = self.w.view(torch.uint8)[perm].contiguous().view(FP8)
            self.interleaved = True
        return self


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


class WeightSource:
    """Produces full (unsharded) tensors by name.  The default draws N(0, std); a checkpoint
    loader can be plugged in through ``loader``."""

    def __init__(self, seed: int = 0, std: float = 0.02, device="cpu",
                 loader: Optional[Callable[[str, Tuple[int, ...]], Optional[torch.Tensor]]] = None,
                 gen_device=None):
        """``gen_device`` is where random tensors are drawn.  The default (CPU) gives the same
        values whatever ``device`` is, so a GPU model and its CPU oracle share weights; drawing on
        the GPU is much faster for full-size benchmark models but yields different values."""
        self.seed, self.std, self.device, self.loader = seed, std, torch.device(device), loader
        self.gen_device = torch.device(gen_device) if gen_device is not None else torch.device("cpu")

    def get(self, name: str, shape: Tuple[int, ...], kind: str = "normal") -> torch.Tensor:
        if self.loader is not None:
            t = self.loader(name, shape)
            if t is not None:
                assert tuple(t.shape) == tuple(shape), (name, t.shape, shape)
                return t.to(self.device, torch.float32)
        if kind == "ones":
            return torch.ones(shape, dtype=torch.float32, device=self.device)
        if kind == "zeros":
            return torch.zeros(shape, dtype=torch.float32, device=self.device)
        g = torch.Generator(device=self.gen_device)
        g.manual_seed(_seed_for(self.seed, name))
        t = torch.randn(shape, dtype=torch.float32, device=self.gen_device, generator=g).to(self.device)
        if kind == "norm":            # norm gains close to one
            return 1.0 + 0.1 * t
        if kind == "bias":
            return 0.1 * t
        return t * self.std


def make_linear(w: torch.Tensor, quant: str, dtype: torch.dtype) -> Linear:
    """Quantise / cast a full-precision [N, K] weight into its runtime form."""
    if quant == "fp8_block" and w.shape[1] % 128 == 0:
        q, s = ref.weight_quant_block(w)
        return Linear(q.contiguous(), s.contiguous())
    return Linear(w.to(dtype).contiguous())


def dequant_linear(lin: Linear) -> torch.Tensor:
    if lin.is_fp8:
        return ref.dequant_block(lin.w, lin.s)
    return lin.w.float()


@dataclass
class KDAWeights:
    """One KDA layer (this rank's heads).  ``w_in`` stacks every projection that reads the layer input, in the
    column order q | k | v | z (output gate) | f_a (low-rank decay gate) | beta, so one GEMM feeds them all."""
    w_in: Linear = None              # [4 Hh D + r + pad(Hh), H]
    f_b: Linear = None               # [Hh D, r]
    conv_w: torch.Tensor = None      # [3 Hh D, 4] fp32
    A_log: torch.Tensor = None       # [Hh] fp32
    dt_bias: torch.Tensor = None     # [Hh D] fp32
    o_norm: torch.Tensor = None      # [D] fp32
    heads: int = 0


@dataclass
class LayerWeights:
    input_norm: torch.Tensor = None
    kda: KDAWeights = None
    post_norm: torch.Tensor = None
    # MLA
    wqkv_a: Linear = None            # [q_lora + kv_lora + rope, H]
    q_norm: torch.Tensor = None
    kv_norm: torch.Tensor = None
    wq_b: Linear = None              # [Hh * qk_head_dim, q_lora]
    w_uk: torch.Tensor = None        # [Hh, nope, kv_lora] (a view of w_uk_t)
    w_uk_t: torch.Tensor = None      # [Hh, kv_lora, nope] contiguous
    w_uv: torch.Tensor = None        # [Hh, v, kv_lora]
    w_kvb: torch.Tensor = None       # [Hh * (nope + v), kv_lora] (CUDA, expanded prefill only)
    wo: Linear = None                # [H, Hh * v]
    # GQA
    wqkv: Linear = None              # [(Hq + 2 Hkv) * D, H]
    bqkv: torch.Tensor = None        # [(Hq + 2 Hkv) * D] projection bias (Qwen2)
    sinks: torch.Tensor = None
    # DSA indexer
    idx_wq: Linear = None            # [Hi * Di, q_lora]
    idx_wk: Linear = None            # [Di, H]
    idx_k_norm_w: torch.Tensor = None
    idx_k_norm_b: torch.Tensor = None
    idx_head_w: torch.Tensor = None  # [Hi, H] head-gate projection
    # dense MLP (also the shared expert of a MoE layer)
    w13: Linear = None               # [2 I, H]
    w2: Linear = None                # [H, I]
    # MoE
    router_w: torch.Tensor = None    # [E, H] fp32
    router_bias: torch.Tensor = None
    shared_gate_w: torch.Tensor = None   # [1, H]: sigmoid gate on the shared expert's output (Qwen2-MoE)
    experts: ExpertWeights = None
    latent_down: Linear = None       # Kimi-K3 LatentMoE  [latent, H]
    latent_up: Linear = None         # [H, latent]
    latent_norm: torch.Tensor = None


@dataclass
class ModelWeights:
    embed: torch.Tensor = None           # [V, H]
    final_norm: torch.Tensor = None
    lm_head: torch.Tensor = None         # [V / tp, H]
    layers: List[LayerWeights] = field(default_factory=list)


def build_weights(cfg: ModelConfig, layout: ParallelLayout, src: WeightSource, dtype: torch.dtype,
                  alias_experts_every: int = 0, experts_on_host: bool = False) -> ModelWeights:
    """Create this rank's weights.  ``alias_experts_every`` > 0 makes MoE layers share physical
    expert storage in a cycle of that many distinct sets (benchmark-only: lets a model whose
    expert bytes exceed HBM run with identical FLOPs and HBM traffic per layer)."""
    H = cfg.hidden_size
    dev = src.device
    quant = cfg.quant if cfg.quant == "fp8_block" else "none"   # mxfp4 applies to the routed experts only
    mw = ModelWeights()
    mw.embed = src.get("model.embed_tokens.weight", (cfg.vocab_size, H)).to(dtype)
    mw.final_norm = src.get("model.norm.weight", (H,), "norm").to(dtype)
    head = mw.embed if cfg.tie_word_embeddings else src.get("lm_head.weight", (cfg.vocab_size, H)).to(dtype)
    if layout.sequence_parallel:
        mw.lm_head = head
    else:
        v0 = layout.tp_rank * cfg.vocab_size // layout.tp_size
        v1 = (layout.tp_rank + 1) * cfg.vocab_size // layout.tp_size
        mw.lm_head = head[v0:v1].contiguous()
    expert_sets: Dict[int, ExpertWeights] = {}
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}"
        lw = LayerWeights()
        lw.input_norm = src.get(f"{p}.input_layernorm.weight", (H,), "norm").to(dtype)
        lw.post_norm = src.get(f"{p}.post_attention_layernorm.weight", (H,), "norm").to(dtype)
        h0, h1 = layout.head_range(cfg.num_heads)
        if cfg.layer_is_kda(l):
            Hk, D, r = cfg.kda_num_heads, cfg.kda_head_dim, cfg.kda_rank
            a0, a1 = layout.head_range(Hk)
            Hh = a1 - a0
            rows = lambda name, n_per: src.get(f"{p}.self_attn.{name}.weight", (Hk * n_per, H)).view(Hk, n_per, H)[a0:a1].reshape(-1, H)
            parts = [rows("q_proj", D), rows("k_proj", D), rows("v_proj", D), rows("g_proj", D),
                     src.get(f"{p}.self_attn.f_a_proj.weight", (r, H)), rows("b_proj", 1)]
            pad = (-Hh) % 8                                  # keep the stacked width a multiple of 8 columns
            if pad:
                parts.append(torch.zeros(pad, H, dtype=torch.float32, device=parts[0].device))
            kw = KDAWeights(heads=Hh)
            kw.w_in = make_linear(torch.cat(parts, 0), "none", dtype)
            fb = src.get(f"{p}.self_attn.f_b_proj.weight", (Hk * D, r)).view(Hk, D, r)[a0:a1].reshape(-1, r)
            kw.f_b = make_linear(fb, "none", dtype)
            conv = [src.get(f"{p}.self_attn.{n}_conv1d.weight", (Hk * D, 4), "bias").view(Hk, D, 4)[a0:a1].reshape(-1, 4)
                    for n in ("q", "k", "v")]
            kw.conv_w = torch.cat(conv, 0).float().contiguous()
            kw.A_log = src.get(f"{p}.self_attn.A_log", (Hk,), "bias")[a0:a1].float().contiguous()
            kw.dt_bias = src.get(f"{p}.self_attn.dt_bias", (Hk * D,), "bias").view(Hk, D)[a0:a1].reshape(-1).float().contiguous()
            kw.o_norm = src.get(f"{p}.self_attn.o_norm.weight", (D,), "norm").float().contiguous()
            wo = src.get(f"{p}.self_attn.o_proj.weight", (H, Hk * D)).view(H, Hk, D)[:, a0:a1].reshape(H, -1)
            lw.wo = make_linear(wo, quant, dtype)
            lw.kda = kw
        elif cfg.is_mla:
            qa = src.get(f"{p}.self_attn.q_a_proj.weight", (cfg.q_lora_rank, H))
            kva = src.get(f"{p}.self_attn.kv_a_proj_with_mqa.weight", (cfg.kv_lora_rank + cfg.qk_rope_head_dim, H))
            lw.wqkv_a = make_linear(torch.cat([qa, kva], 0), quant, dtype)
            lw.q_norm = src.get(f"{p}.self_attn.q_a_layernorm.weight", (cfg.q_lora_rank,), "norm").to(dtype)
            lw.kv_norm = src.get(f"{p}.self_attn.kv_a_layernorm.weight", (cfg.kv_lora_rank,), "norm").to(dtype)
            qb = src.get(f"{p}.self_attn.q_b_proj.weight", (cfg.num_heads * cfg.qk_head_dim, cfg.q_lora_rank))
            qb = qb.view(cfg.num_heads, cfg.qk_head_dim, cfg.q_lora_rank)[h0:h1].reshape(-1, cfg.q_lora_rank)
            lw.wq_b = make_linear(qb, quant, dtype)
            kvb = src.get(f"{p}.self_attn.kv_b_proj.weight",
                          (cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank))
            kvb = kvb.view(cfg.num_heads, cfg.qk_nope_head_dim + cfg.v_head_dim, cfg.kv_lora_rank)[h0:h1]
            # W_UK is kept transposed ([heads, kv_lora, nope]: the K-major operand of the absorb kernel);
            # w_uk is a view of the same storage in the [heads, nope, kv_lora] form
            lw.w_uk_t = kvb[:, : cfg.qk_nope_head_dim].transpose(1, 2).contiguous().to(dtype)
            lw.w_uk = lw.w_uk_t.transpose(1, 2)
            lw.w_uv = kvb[:, cfg.qk_nope_head_dim:].contiguous().to(dtype)
            if str(dev).startswith("cuda") and cfg.qk_nope_head_dim == 128 and cfg.v_head_dim == 128 \
                    and cfg.qk_rope_head_dim == 64 and not cfg.has_dsa:
                # whole kv_b ([heads * (nope + v), kv_lora]) for the expanded prefill attention
                lw.w_kvb = kvb.reshape(-1, cfg.kv_lora_rank).contiguous().to(dtype)
            wo = src.get(f"{p}.self_attn.o_proj.weight", (H, cfg.num_heads * cfg.v_head_dim))
            wo = wo.view(H, cfg.num_heads, cfg.v_head_dim)[:, h0:h1].reshape(H, -1)
            lw.wo = make_linear(wo, quant, dtype)
            if cfg.layer_has_indexer(l):
                Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                lw.idx_wq = make_linear(src.get(f"{p}.self_attn.indexer.wq_b.weight", (Hi * Di, cfg.q_lora_rank)),
                                        "none", dtype)
                lw.idx_wk = make_linear(src.get(f"{p}.self_attn.indexer.wk.weight", (Di, H)), "none", dtype)
                lw.idx_k_norm_w = src.get(f"{p}.self_attn.indexer.k_norm.weight", (Di,), "norm").to(dtype)
                lw.idx_k_norm_b = src.get(f"{p}.self_attn.indexer.k_norm.bias", (Di,), "bias").to(dtype)
                lw.idx_head_w = src.get(f"{p}.self_attn.indexer.weights_proj.weight", (Hi, H)).to(dtype)
        else:
            D, Hq, Hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
            k0, k1 = layout.head_range(Hkv)
            wq = src.get(f"{p}.self_attn.q_proj.weight", (Hq * D, H)).view(Hq, D, H)[h0:h1].reshape(-1, H)
            wk = src.get(f"{p}.self_attn.k_proj.weight", (Hkv * D, H)).view(Hkv, D, H)[k0:k1].reshape(-1, H)
            wv = src.get(f"{p}.self_attn.v_proj.weight", (Hkv * D, H)).view(Hkv, D, H)[k0:k1].reshape(-1, H)
            lw.wqkv = make_linear(torch.cat([wq, wk, wv], 0), quant, dtype)
            if cfg.attention_bias:
                bq = src.get(f"{p}.self_attn.q_proj.bias", (Hq * D,), "bias").view(Hq, D)[h0:h1].reshape(-1)
                bk = src.get(f"{p}.self_attn.k_proj.bias", (Hkv * D,), "bias").view(Hkv, D)[k0:k1].reshape(-1)
                bv = src.get(f"{p}.self_attn.v_proj.bias", (Hkv * D,), "bias").view(Hkv, D)[k0:k1].reshape(-1)
                lw.bqkv = torch.cat([bq, bk, bv], 0).to(dtype).contiguous()
            wo = src.get(f"{p}.self_attn.o_proj.weight", (H, Hq * D)).view(H, Hq, D)[:, h0:h1].reshape(H, -1)
            lw.wo = make_linear(wo, quant, dtype)
            if cfg.attention_sinks:
                lw.sinks = src.get(f"{p}.self_attn.sinks", (Hq,), "bias")[h0:h1].contiguous()

        def mlp_pair(prefix: str, inter: int, hid: int, shard: bool = True):
            i0, i1 = 0, inter
            if shard:
                i0, i1 = layout.tp_rank * inter // layout.tp_size, (layout.tp_rank + 1) * inter // layout.tp_size
            g = src.get(f"{prefix}.gate_proj.weight", (inter, hid))[i0:i1]
            u = src.get(f"{prefix}.up_proj.weight", (inter, hid))[i0:i1]
            d = src.get(f"{prefix}.down_proj.weight", (hid, inter))[:, i0:i1]
            return (make_linear(torch.cat([g, u], 0), quant, dtype).interleave_gate_up_(),
                    make_linear(d.contiguous(), quant, dtype))

        if cfg.is_moe_layer(l):
            E, I, eh = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.expert_hidden
            lw.router_w = src.get(f"{p}.mlp.gate.weight", (E, H)).float()
            if cfg.scoring_func in ("sigmoid", "sqrtsoftplus"):
                lw.router_bias = src.get(f"{p}.mlp.gate.e_score_correction_bias", (E,), "bias").float()
            if cfg.shared_expert_gate:
                lw.shared_gate_w = src.get(f"{p}.mlp.shared_expert_gate.weight", (1, H)).to(dtype)
            if cfg.moe_latent_size:
                lw.latent_down = make_linear(src.get(f"{p}.mlp.latent_down_proj.weight", (eh, H)), "none", dtype)
                lw.latent_up = make_linear(src.get(f"{p}.mlp.latent_up_proj.weight", (H, eh)), "none", dtype)
                lw.latent_norm = src.get(f"{p}.mlp.latent_norm.weight", (eh,), "norm").to(dtype)
            key = (l - cfg.first_k_dense) % alias_experts_every if alias_experts_every else l
            if key in expert_sets:
                lw.experts = expert_sets[key]
            else:
                e0, e1 = layout.expert_range(E)
                w13s, w2s, s13, s2 = [], [], [], []
                equant = "fp8_block" if quant == "fp8_block" else "none"
                if cfg.quant in ("mxfp4", "int4") and eh % 64 == 0 and I % 64 == 0:
                    if cfg.quant == "mxfp4":
                        from ..ops.mxfp4 import quantize as quantize_w4
                    else:
                        from ..ops.int4 import quantize as quantize_w4
                    for e in range(e0, e1):
                        ep = f"{p}.mlp.experts.{e}"
                        g = src.get(f"{ep}.gate_proj.weight", (I, eh))
                        u = src.get(f"{ep}.up_proj.weight", (I, eh))
                        d = src.get(f"{ep}.down_proj.weight", (eh, I))
                        q13, sc13 = quantize_w4(torch.cat([g, u], 0))
                        q2, sc2 = quantize_w4(d)
                        w13s.append(q13); s13.append(sc13); w2s.append(q2); s2.append(sc2)
                    lw.experts = ExpertWeights(w13=torch.stack(w13s), w2=torch.stack(w2s), w13_s=torch.stack(s13),
                                               w2_s=torch.stack(s2), quant=cfg.quant,
                                               activation=cfg.activation).to_device_layout()
                    expert_sets[key] = lw.experts
                for e in (range(e0, e1) if key not in expert_sets else ()):
                    ep = f"{p}.mlp.experts.{e}"
                    g = src.get(f"{ep}.gate_proj.weight", (I, eh))
                    u = src.get(f"{ep}.up_proj.weight", (I, eh))
                    d = src.get(f"{ep}.down_proj.weight", (eh, I))
                    a = make_linear(torch.cat([g, u], 0), equant, dtype)
                    b = make_linear(d, equant, dtype)
                    w13s.append(a.w); w2s.append(b.w)
                    if a.is_fp8:
                        s13.append(a.s); s2.append(b.s)
                if key not in expert_sets:
                    lw.experts = ExpertWeights(
                        w13=torch.stack(w13s), w2=torch.stack(w2s),
                        w13_s=torch.stack(s13) if s13 else None, w2_s=torch.stack(s2) if s2 else None,
                        quant=equant, activation=cfg.activation).to_device_layout()
                    expert_sets[key] = lw.experts
            if experts_on_host and lw.experts.w13.is_cuda:
                # streamed models never hold all layers' experts on the GPU: park each set on the host at once
                e = lw.experts
                for f in ("w13", "w2", "w13_s", "w2_s"):
                    if getattr(e, f) is not None:
                        setattr(e, f, getattr(e, f).cpu())
            if cfg.n_shared_experts:
                lw.w13, lw.w2 = mlp_pair(f"{p}.mlp.shared_experts", I * cfg.n_shared_experts, H,
                                         shard=not layout.sequence_parallel)
        else:
            lw.w13, lw.w2 = mlp_pair(f"{p}.mlp", cfg.intermediate_size, H)
        mw.layers.append(lw)
    return mw


def checkpoint_tensor_specs(cfg: ModelConfig):
    """(name, shape, init kind, layer) of every checkpoint tensor of an MLA model, in file order
    (layer -1 = embeddings / final norm / lm_head)."""
    H = cfg.hidden_size
    out = [("model.embed_tokens.weight", (cfg.vocab_size, H), "normal", -1),
           ("model.norm.weight", (H,), "norm", -1)]
    if not cfg.tie_word_embeddings:
        out.append(("lm_head.weight", (cfg.vocab_size, H), "normal", -1))
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}"
        a = f"{p}.self_attn"
        out += [(f"{p}.input_layernorm.weight", (H,), "norm", l),
                (f"{p}.post_attention_layernorm.weight", (H,), "norm", l)]
        if cfg.is_mla:
            out += [(f"{a}.q_a_proj.weight", (cfg.q_lora_rank, H), "normal", l),
                    (f"{a}.kv_a_proj_with_mqa.weight", (cfg.kv_lora_rank + cfg.qk_rope_head_dim, H), "normal", l),
                    (f"{a}.q_a_layernorm.weight", (cfg.q_lora_rank,), "norm", l),
                    (f"{a}.kv_a_layernorm.weight", (cfg.kv_lora_rank,), "norm", l),
                    (f"{a}.q_b_proj.weight", (cfg.num_heads * cfg.qk_head_dim, cfg.q_lora_rank), "normal", l),
                    (f"{a}.kv_b_proj.weight", (cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank),
                     "normal", l),
                    (f"{a}.o_proj.weight", (H, cfg.num_heads * cfg.v_head_dim), "normal", l)]
            if cfg.layer_has_indexer(l):
                Hi, Di = cfg.index_n_heads, cfg.index_head_dim
                out += [(f"{a}.indexer.wq_b.weight", (Hi * Di, cfg.q_lora_rank), "normal", l),
                        (f"{a}.indexer.wk.weight", (Di, H), "normal", l),
                        (f"{a}.indexer.k_norm.weight", (Di,), "norm", l),
                        (f"{a}.indexer.k_norm.bias", (Di,), "bias", l),
                        (f"{a}.indexer.weights_proj.weight", (Hi, H), "normal", l)]
        else:
            D, Hq, Hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
            out += [(f"{a}.q_proj.weight", (Hq * D, H), "normal", l), (f"{a}.k_proj.weight", (Hkv * D, H), "normal", l),
                    (f"{a}.v_proj.weight", (Hkv * D, H), "normal", l), (f"{a}.o_proj.weight", (H, Hq * D), "normal", l)]
            if cfg.attention_bias:
                out += [(f"{a}.q_proj.bias", (Hq * D,), "bias", l), (f"{a}.k_proj.bias", (Hkv * D,), "bias", l),
                        (f"{a}.v_proj.bias", (Hkv * D,), "bias", l)]
            if cfg.attention_sinks:
                out.append((f"{a}.sinks", (Hq,), "bias", l))

        def mlp(prefix, inter, hid):
            return [(f"{prefix}.gate_proj.weight", (inter, hid), "normal", l),
                    (f"{prefix}.up_proj.weight", (inter, hid), "normal", l),
                    (f"{prefix}.down_proj.weight", (hid, inter), "normal", l)]

        if cfg.is_moe_layer(l):
            E, I, eh = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.expert_hidden
            out.append((f"{p}.mlp.gate.weight", (E, H), "normal", l))
            if cfg.scoring_func in ("sigmoid", "sqrtsoftplus"):
                out.append((f"{p}.mlp.gate.e_score_correction_bias", (E,), "bias", l))
            if cfg.shared_expert_gate:
                out.append((f"{p}.mlp.shared_expert_gate.weight", (1, H), "normal", l))
            if cfg.moe_latent_size:
                out += [(f"{p}.mlp.latent_down_proj.weight", (eh, H), "normal", l),
                        (f"{p}.mlp.latent_up_proj.weight", (H, eh), "normal", l),
                        (f"{p}.mlp.latent_norm.weight", (eh,), "norm", l)]
            for e in range(E):
                out += mlp(f"{p}.mlp.experts.{e}", I, eh)
            if cfg.n_shared_experts:
                out += mlp(f"{p}.mlp.shared_experts", I * cfg.n_shared_experts, H)
        else:
            out += mlp(f"{p}.mlp", cfg.intermediate_size, H)
    return out
