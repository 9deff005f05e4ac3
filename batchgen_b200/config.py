"""Model and engine configuration.

One ``ModelConfig`` describes every supported family; fields that a family does not use
keep their neutral default (``index_topk == 0`` means no DSA indexer, ``moe_latent_size == 0``
means experts work in the hidden size, ``num_kv_heads > 0`` selects GQA instead of MLA).

Reference parity: the reference spreads this over per-model ``config.py`` / planner files and
``batchgen/config/config.py:26-293`` (engine config dataclasses + JSON parser) and identifies
models through ``batchgen/config/model_registry.py:60-117``.  Here a single registry maps model
names (and HF-style ids) to presets.
"""
from __future__ import annotations

import dataclasses
import json
import math
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class ModelConfig:
    name: str = "tiny-deepseek-v3"
    family: str = "deepseek_v3"  # deepseek_v3 | deepseek_v2 | deepseek_v4 | glm5 | kimi_k3 | kimi_k25 | gpt_oss | minimax | mixtral | qwen2_moe
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 2
    first_k_dense: int = 1
    intermediate_size: int = 512          # dense MLP intermediate
    moe_intermediate_size: int = 128      # routed / shared expert intermediate
    n_routed_experts: int = 8
    n_shared_experts: int = 1
    num_experts_per_tok: int = 2
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = True
    scoring_func: str = "sigmoid"          # sigmoid | softmax (over the selected) | softmax_all | sqrtsoftplus
    shared_expert_gate: bool = False       # Qwen2-MoE: the shared expert's output is scaled by sigmoid(x . w_gate)
    moe_latent_size: int = 0               # Kimi-K3 LatentMoE: experts run in this width
    activation: str = "silu"               # silu | swiglu_clamped (GPT-OSS)
    # ---- attention: MLA
    num_heads: int = 4
    q_lora_rank: int = 128
    kv_lora_rank: int = 64
    qk_nope_head_dim: int = 32
    qk_rope_head_dim: int = 16
    v_head_dim: int = 32
    # ---- attention: GQA (used when num_kv_heads > 0)
    num_kv_heads: int = 0
    head_dim: int = 0
    sliding_window: int = 0
    attention_sinks: bool = False
    attention_bias: bool = False           # GQA: q/k/v projections carry a bias (Qwen2)
    # ---- rope
    rope_theta: float = 10000.0
    rope_interleaved: bool = True
    rope_scaling_factor: float = 1.0       # YaRN factor (1 = off)
    rope_original_max_pos: int = 4096
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_mscale: float = 1.0
    rope_mscale_all_dim: float = 0.0
    max_position_embeddings: int = 163840
    rms_eps: float = 1e-6
    # ---- DSA sparse-attention indexer (GLM-5.x / Kimi-K3.1)
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    indexer_full_layers: Tuple[int, ...] = ()   # layers that own an indexer; others reuse
    # ---- KDA linear-attention layers (Kimi-Linear / Kimi-K3): those layers keep a recurrent state per
    # sequence instead of paged KV; the other layers are MLA
    kda_layers: Tuple[int, ...] = ()
    kda_num_heads: int = 0
    kda_head_dim: int = 128
    kda_gate_rank: int = 0                 # width of the low-rank decay-gate projection (0 = head dim)
    # ---- DeepSeek-V4: one latent KV head shared by all query heads (K = V), a sliding window of raw KV plus one
    # pooled entry per ``compress_ratios[layer]`` tokens (0 = window only; 4 = overlapped windows + top-k indexer),
    # grouped low-rank output projection, hyper-connection residual streams, hash-routed first layers
    compress_ratios: Tuple[int, ...] = ()
    compress_rope_theta: float = 0.0
    o_groups: int = 0
    o_lora_rank: int = 0
    hc_mult: int = 0
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    num_hash_layers: int = 0
    swiglu_limit: float = 0.0
    # ---- quantisation of linear / expert weights
    quant: str = "none"                    # none | fp8_block | mxfp4 | int4
    quant_block: int = 128
    # ---- misc
    eos_token_id: int = 1
    bos_token_id: int = 0
    tie_word_embeddings: bool = False

    # derived ------------------------------------------------------------------
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def is_v4(self) -> bool:
        return len(self.compress_ratios) > 0

    def v4_state_floats_per_seq(self) -> int:
        """fp32 words of per-sequence state of a DeepSeek-V4 model: per layer the window ring, the compressor's
        pending window(s) of projections and gate scores, and the same for the indexer's compressor."""
        n, D, Di, win = 0, self.head_dim, self.index_head_dim, self.sliding_window
        for r in self.compress_ratios:
            n += win * D
            if r:
                c = 2 if r == 4 else 1
                n += 2 * (c * r) * (c * D)
                if r == 4:
                    n += 2 * (2 * r) * (2 * Di)
        return n

    @property
    def kv_cache_dim(self) -> int:
        """Width of one cached latent row (normalised c_kv followed by roped k_pe)."""
        if self.is_v4:
            return self.head_dim
        if self.num_kv_heads > 0:
            return 2 * self.num_kv_heads * self.head_dim
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def is_mla(self) -> bool:
        return self.num_kv_heads == 0

    @property
    def has_dsa(self) -> bool:
        return self.index_topk > 0 and not self.is_v4

    @property
    def expert_hidden(self) -> int:
        return self.moe_latent_size or self.hidden_size

    @property
    def softmax_scale(self) -> float:
        d = self.qk_head_dim if self.is_mla else self.head_dim
        scale = d ** -0.5
        if self.rope_scaling_factor > 1.0 and self.rope_mscale_all_dim:
            m = 0.1 * self.rope_mscale_all_dim * math.log(self.rope_scaling_factor) + 1.0
            scale = scale * m * m
        return scale

    @property
    def has_kda(self) -> bool:
        return len(self.kda_layers) > 0

    def layer_is_kda(self, layer: int) -> bool:
        return layer in self.kda_layers

    @property
    def kda_rank(self) -> int:
        return self.kda_gate_rank or self.kda_head_dim

    def kda_state_bytes_per_seq(self, tp_size: int = 1) -> int:
        """Recurrent state (fp32 [H, D, D]) plus convolution windows (fp32 [3 H D, 3]) of all KDA layers."""
        h, d = self.kda_num_heads // tp_size, self.kda_head_dim
        return len(self.kda_layers) * 4 * (h * d * d + 9 * h * d)

    def is_moe_layer(self, layer: int) -> bool:
        return self.n_routed_experts > 0 and layer >= self.first_k_dense

    def layer_has_indexer(self, layer: int) -> bool:
        if not self.has_dsa:
            return False
        return (not self.indexer_full_layers) or layer in self.indexer_full_layers

    def kv_bytes_per_token(self, kv_dtype_bytes: int = 2) -> int:
        if self.is_v4:
            # paged part only (pooled entries and their index keys); the window and compressor state is per sequence
            b = 0.0
            for r in self.compress_ratios:
                if r:
                    b += self.head_dim * kv_dtype_bytes / r
                    if r == 4:
                        b += self.index_head_dim * kv_dtype_bytes / r
            return int(math.ceil(b))
        b = (self.num_layers - len(self.kda_layers)) * self.kv_cache_dim * kv_dtype_bytes
        if self.has_dsa:
            n_idx = len(self.indexer_full_layers) or self.num_layers
            b += n_idx * (self.index_head_dim + 4)  # e4m3 keys + fp32 scale per token
        return b

    def param_count(self) -> int:
        h = self.hidden_size
        n = 2 * self.vocab_size * h
        if self.is_v4:
            D, Di = self.head_dim, self.index_head_dim
            for l, r in enumerate(self.compress_ratios):
                n += h * self.q_lora_rank + self.q_lora_rank * self.num_heads * D + h * D
                n += self.num_heads * D * self.o_lora_rank + self.o_groups * self.o_lora_rank * h
                if r:
                    c = 2 if r == 4 else 1
                    n += 2 * h * c * D
                    if r == 4:
                        n += self.q_lora_rank * self.index_n_heads * Di + h * self.index_n_heads + 4 * h * Di
                n += 3 * h * self.moe_intermediate_size * (self.n_routed_experts + self.n_shared_experts)
                n += h * self.n_routed_experts + 2 * (2 + self.hc_mult) * self.hc_mult * self.hc_mult * h
            return n
        for l in range(self.num_layers):
            if self.layer_is_kda(l):
                hd = self.kda_num_heads * self.kda_head_dim
                n += h * (4 * hd + self.kda_num_heads + self.kda_rank) + self.kda_rank * hd + hd * h
            elif self.is_mla:
                n += h * self.q_lora_rank + self.q_lora_rank * self.num_heads * self.qk_head_dim
                n += h * self.kv_cache_dim
                n += self.kv_lora_rank * self.num_heads * (self.qk_nope_head_dim + self.v_head_dim)
                n += self.num_heads * self.v_head_dim * h
            else:
                n += h * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
                n += self.num_heads * self.head_dim * h
            if self.is_moe_layer(l):
                eh = self.expert_hidden
                n += 3 * eh * self.moe_intermediate_size * (self.n_routed_experts + self.n_shared_experts)
                n += h * self.n_routed_experts
            else:
                n += 3 * h * self.intermediate_size
        return n

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1)

    @classmethod
    def from_dict(cls, d: Dict) -> "ModelConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in d.items() if k in names}
        if "kda_layers" in kw:
            kw["kda_layers"] = tuple(kw["kda_layers"])
        if "indexer_full_layers" in kw:
            kw["indexer_full_layers"] = tuple(kw["indexer_full_layers"])
        if "compress_ratios" in kw:
            kw["compress_ratios"] = tuple(kw["compress_ratios"])
        return cls(**kw)


# ------------------------------------------------------------------ presets
def tiny_deepseek_v3() -> ModelConfig:
    """The CPU fp32 correctness model: 2 layers (dense, MoE), hidden 256, 8 experts top-2."""
    return ModelConfig()


def tiny_glm5() -> ModelConfig:
    return ModelConfig(name="tiny-glm5", family="glm5", num_layers=3, first_k_dense=1,
                       index_n_heads=4, index_head_dim=32, index_topk=16,
                       indexer_full_layers=(0, 2), rope_interleaved=True,
                       routed_scaling_factor=2.5)


def tiny_kimi_k3() -> ModelConfig:
    return ModelConfig(name="tiny-kimi-k3", family="kimi_k3", num_layers=2, first_k_dense=0,
                       n_routed_experts=16, num_experts_per_tok=4, moe_latent_size=128,
                       moe_intermediate_size=64, quant="none")


def tiny_kimi_linear() -> ModelConfig:
    """Three KDA layers to one MLA layer, as in Kimi-Linear; LatentMoE off."""
    return ModelConfig(name="tiny-kimi-linear", family="kimi_k3", num_layers=4, first_k_dense=1,
                       n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                       kda_layers=(0, 1, 2), kda_num_heads=2, kda_head_dim=64, kda_gate_rank=32)


def tiny_kimi_k31() -> ModelConfig:
    """KDA layers plus an MLA layer that carries a DSA indexer (the Kimi-K3.1 arrangement)."""
    import dataclasses
    return dataclasses.replace(tiny_kimi_linear(), name="tiny-kimi-k3.1", index_n_heads=4, index_head_dim=32,
                               index_topk=16, indexer_full_layers=(3,))


def tiny_gpt_oss() -> ModelConfig:
    return ModelConfig(name="tiny-gpt-oss", family="gpt_oss", num_layers=2, first_k_dense=0,
                       num_heads=8, num_kv_heads=2, head_dim=32, sliding_window=16,
                       attention_sinks=True, scoring_func="softmax", n_shared_experts=0,
                       n_routed_experts=8, num_experts_per_tok=2, activation="swiglu_clamped",
                       rope_interleaved=False)


def tiny_minimax() -> ModelConfig:
    """MiniMax-shaped GQA + FP8 MoE at the smallest geometry the GPU kernels tile (head_dim 128, hidden 1024)."""
    return ModelConfig(name="tiny-minimax", family="minimax", vocab_size=4096, hidden_size=1024, num_layers=2,
                       first_k_dense=0, moe_intermediate_size=512, n_routed_experts=16, n_shared_experts=0,
                       num_experts_per_tok=4, num_heads=16, num_kv_heads=4, head_dim=128, rope_interleaved=False,
                       quant="fp8_block")


def tiny_gpt_oss_64() -> ModelConfig:
    """GPT-OSS-shaped GQA (head_dim 64, sinks, sliding window on alternate layers) at kernel-sized geometry."""
    return ModelConfig(name="tiny-gpt-oss-64", family="gpt_oss", vocab_size=4096, hidden_size=1024, num_layers=2,
                       first_k_dense=0, moe_intermediate_size=512, n_routed_experts=16, n_shared_experts=0,
                       num_experts_per_tok=4, num_heads=16, num_kv_heads=4, head_dim=64, sliding_window=128,
                       attention_sinks=True, scoring_func="softmax", activation="swiglu_clamped",
                       rope_interleaved=False)


def tiny_deepseek_v2() -> ModelConfig:
    """DeepSeek-V2 routing at toy size: softmax over all experts, groups ranked by their best expert, weights not
    renormalised, two shared experts."""
    return ModelConfig(name="tiny-deepseek-v2", family="deepseek_v2", num_layers=2, first_k_dense=1,
                       n_routed_experts=16, n_shared_experts=2, num_experts_per_tok=4, n_group=4, topk_group=2,
                       scoring_func="softmax_all", norm_topk_prob=False, routed_scaling_factor=4.0,
                       moe_intermediate_size=64)


def tiny_mixtral() -> ModelConfig:
    return ModelConfig(name="tiny-mixtral", family="mixtral", num_layers=2, first_k_dense=0, num_heads=8,
                       num_kv_heads=2, head_dim=32, scoring_func="softmax", n_shared_experts=0, n_routed_experts=8,
                       num_experts_per_tok=2, rope_interleaved=False, rope_theta=1e6)


def tiny_qwen2_moe() -> ModelConfig:
    """Qwen2-MoE at toy size: biased q/k/v, softmax over all experts without renormalisation, gated shared expert."""
    return ModelConfig(name="tiny-qwen2-moe", family="qwen2_moe", num_layers=2, first_k_dense=0, num_heads=8,
                       num_kv_heads=2, head_dim=32, attention_bias=True, scoring_func="softmax_all",
                       norm_topk_prob=False, n_shared_experts=2, shared_expert_gate=True, n_routed_experts=8,
                       num_experts_per_tok=2, moe_intermediate_size=64, rope_interleaved=False, rope_theta=1e6)


def deepseek_v2_236b() -> ModelConfig:
    """DeepSeek-V2 (236B): the MLA + MoE generation before V3 (reference: batchgen/models/deepseek/deepseekv2/config_v2.json)."""
    return ModelConfig(
        name="deepseek-v2", family="deepseek_v2", vocab_size=102400, hidden_size=5120, num_layers=60,
        first_k_dense=1, intermediate_size=12288, moe_intermediate_size=1536, n_routed_experts=160,
        n_shared_experts=2, num_experts_per_tok=6, n_group=8, topk_group=3, routed_scaling_factor=16.0,
        norm_topk_prob=False, scoring_func="softmax_all", num_heads=128, q_lora_rank=1536, kv_lora_rank=512,
        qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rope_theta=10000.0, rope_scaling_factor=40.0,
        rope_original_max_pos=4096, rope_mscale=0.707, rope_mscale_all_dim=0.707, eos_token_id=100001,
        bos_token_id=100000)


def mixtral_8x7b() -> ModelConfig:
    """Mixtral-8x7B (reference: batchgen/models/mixtral/config.py)."""
    return ModelConfig(
        name="mixtral-8x7b", family="mixtral", vocab_size=32000, hidden_size=4096, num_layers=32, first_k_dense=0,
        moe_intermediate_size=14336, n_routed_experts=8, n_shared_experts=0, num_experts_per_tok=2,
        scoring_func="softmax", num_heads=32, num_kv_heads=8, head_dim=128, rope_theta=1e6, rope_interleaved=False,
        max_position_embeddings=32768, rms_eps=1e-5, eos_token_id=2, bos_token_id=1)


def mixtral_8x22b() -> ModelConfig:
    import dataclasses
    return dataclasses.replace(mixtral_8x7b(), name="mixtral-8x22b", hidden_size=6144, num_layers=56,
                               moe_intermediate_size=16384, num_heads=48, max_position_embeddings=65536)


def qwen2_57b_a14b() -> ModelConfig:
    """Qwen2-57B-A14B, the Qwen2-MoE checkpoint family the reference's Qwen initializer serves
    (batchgen/models/Qwen_Initializer.py)."""
    return ModelConfig(
        name="qwen2-57b-a14b", family="qwen2_moe", vocab_size=151936, hidden_size=3584, num_layers=28,
        first_k_dense=0, moe_intermediate_size=2560, n_routed_experts=64, n_shared_experts=8,
        shared_expert_gate=True, num_experts_per_tok=8, scoring_func="softmax_all", norm_topk_prob=False,
        num_heads=28, num_kv_heads=4, head_dim=128, attention_bias=True, rope_theta=1e6, rope_interleaved=False,
        max_position_embeddings=65536, eos_token_id=151643, bos_token_id=151643)


def qwen15_moe_a27b() -> ModelConfig:
    return ModelConfig(
        name="qwen1.5-moe-a2.7b", family="qwen2_moe", vocab_size=151936, hidden_size=2048, num_layers=24,
        first_k_dense=0, moe_intermediate_size=1408, n_routed_experts=60, n_shared_experts=4,
        shared_expert_gate=True, num_experts_per_tok=4, scoring_func="softmax_all", norm_topk_prob=False,
        num_heads=16, num_kv_heads=16, head_dim=128, attention_bias=True, rope_theta=1e6, rope_interleaved=False,
        max_position_embeddings=8192, eos_token_id=151643, bos_token_id=151643)


def tiny_deepseek_v4() -> ModelConfig:
    """DeepSeek-V4 at toy size: a window-only layer, an overlapped ratio-4 layer with its indexer, and a ratio-8
    layer; the first layer routes by token id."""
    return ModelConfig(name="tiny-deepseek-v4", family="deepseek_v4", vocab_size=512, hidden_size=128, num_layers=3,
                       first_k_dense=0, moe_intermediate_size=64, n_routed_experts=8, n_shared_experts=1,
                       num_experts_per_tok=2, scoring_func="sqrtsoftplus", routed_scaling_factor=1.5,
                       num_heads=4, head_dim=64, q_lora_rank=64, qk_rope_head_dim=16, sliding_window=8,
                       compress_ratios=(0, 4, 8), compress_rope_theta=160000.0, rope_scaling_factor=4.0,
                       rope_original_max_pos=64, o_groups=2, o_lora_rank=32, hc_mult=2, hc_sinkhorn_iters=4,
                       num_hash_layers=1, swiglu_limit=10.0, index_n_heads=8, index_head_dim=32, index_topk=4)


def _v4_ratios(head: Tuple[int, ...], n_layers: int) -> Tuple[int, ...]:
    rest = n_layers - len(head)
    return head + tuple(4 if i % 2 == 0 else 128 for i in range(rest))


def deepseek_v4_flash() -> ModelConfig:
    """DeepSeek-V4-Flash (reference: batchgen/models/deepseek/deepseekv4_flash/config.py:36-119)."""
    return ModelConfig(
        name="deepseek-v4-flash", family="deepseek_v4", vocab_size=129280, hidden_size=4096, num_layers=43,
        first_k_dense=0, moe_intermediate_size=2048, n_routed_experts=256, n_shared_experts=1,
        num_experts_per_tok=6, scoring_func="sqrtsoftplus", routed_scaling_factor=1.5, norm_topk_prob=True,
        num_heads=64, head_dim=512, q_lora_rank=1024, qk_rope_head_dim=64, sliding_window=128,
        compress_ratios=_v4_ratios((0, 0), 43), compress_rope_theta=160000.0, rope_theta=10000.0,
        rope_scaling_factor=16.0, rope_original_max_pos=65536, o_groups=8, o_lora_rank=1024, hc_mult=4,
        hc_sinkhorn_iters=20, num_hash_layers=3, swiglu_limit=10.0, index_n_heads=64, index_head_dim=128,
        index_topk=512, max_position_embeddings=1048576, quant="mxfp4", quant_block=32, eos_token_id=1,
        bos_token_id=0)


def deepseek_v4_pro() -> ModelConfig:
    import dataclasses
    return dataclasses.replace(
        deepseek_v4_flash(), name="deepseek-v4-pro", hidden_size=7168, num_layers=61, moe_intermediate_size=3072,
        n_routed_experts=384, routed_scaling_factor=2.5, num_heads=128, q_lora_rank=1536, o_groups=16,
        compress_ratios=_v4_ratios((128, 128), 61), index_topk=1024)


def deepseek_v3_671b() -> ModelConfig:
    return ModelConfig(
        name="deepseek-v3-671b", family="deepseek_v3", vocab_size=129280, hidden_size=7168,
        num_layers=61, first_k_dense=3, intermediate_size=18432, moe_intermediate_size=2048,
        n_routed_experts=256, n_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4,
        routed_scaling_factor=2.5, norm_topk_prob=True, num_heads=128, q_lora_rank=1536,
        kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
        rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_max_pos=4096,
        rope_mscale=1.0, rope_mscale_all_dim=1.0, quant="fp8_block", eos_token_id=1)


def glm5_3() -> ModelConfig:
    full = tuple(sorted(set(list(range(0, 78, 4)) + [77])))[:21]
    return ModelConfig(
        name="glm-5.3-fp8", family="glm5", vocab_size=154880, hidden_size=6144, num_layers=78,
        first_k_dense=3, intermediate_size=12288, moe_intermediate_size=2048,
        n_routed_experts=256, n_shared_experts=1, num_experts_per_tok=8, n_group=1, topk_group=1,
        routed_scaling_factor=2.5, num_heads=64, q_lora_rank=2048, kv_lora_rank=512,
        qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256, rope_theta=1000000.0,
        rope_interleaved=True, index_n_heads=32, index_head_dim=128, index_topk=2048,
        indexer_full_layers=full, quant="fp8_block", max_position_embeddings=1048576)


def kimi_k3() -> ModelConfig:
    return ModelConfig(
        name="kimi-k3", family="kimi_k3", vocab_size=163840, hidden_size=7168, num_layers=93,
        first_k_dense=1, intermediate_size=18432, moe_intermediate_size=3072,
        n_routed_experts=896, n_shared_experts=1, num_experts_per_tok=16, n_group=1,
        topk_group=1, routed_scaling_factor=2.5, moe_latent_size=3584, num_heads=64,
        q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
        v_head_dim=128, quant="mxfp4", quant_block=32)


def kimi_k3_kda() -> ModelConfig:
    """Kimi-K3 with its linear-attention layers: of the 93 layers every fourth (24 in all) is NoPE-MLA,
    the other 69 are KDA (64 heads of 128)."""
    import dataclasses
    mla = set(range(3, 93, 4)) | {92}
    return dataclasses.replace(kimi_k3(), name="kimi-k3-kda", kda_layers=tuple(l for l in range(93) if l not in mla),
                               kda_num_heads=64, kda_head_dim=128)


def kimi_k31() -> ModelConfig:
    """Kimi-K3.1: K3 with KDA layers and a DSA indexer (top-2048, 32 heads of 128) on every MLA layer."""
    import dataclasses
    base = kimi_k3_kda()
    mla = tuple(l for l in range(base.num_layers) if l not in base.kda_layers)
    return dataclasses.replace(base, name="kimi-k3.1", index_n_heads=32, index_head_dim=128, index_topk=2048,
                               indexer_full_layers=mla)


def kimi_linear_48b() -> ModelConfig:
    return ModelConfig(
        name="kimi-linear-48b", family="kimi_k3", vocab_size=163840, hidden_size=2304, num_layers=27,
        first_k_dense=1, intermediate_size=9216, moe_intermediate_size=1024, n_routed_experts=256,
        n_shared_experts=1, num_experts_per_tok=8, routed_scaling_factor=2.446, num_heads=32,
        q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
        kda_layers=tuple(l for l in range(27) if l % 4 != 3), kda_num_heads=32, kda_head_dim=128)


def kimi_k25() -> ModelConfig:
    return ModelConfig(
        name="kimi-k2.5", family="kimi_k25", vocab_size=163840, hidden_size=7168, num_layers=61,
        first_k_dense=1, intermediate_size=18432, moe_intermediate_size=2048,
        n_routed_experts=384, n_shared_experts=1, num_experts_per_tok=8, routed_scaling_factor=2.827,
        num_heads=64, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
        qk_rope_head_dim=64, v_head_dim=128, quant="mxfp4", quant_block=32)


def gpt_oss_120b() -> ModelConfig:
    return ModelConfig(
        name="gpt-oss-120b", family="gpt_oss", vocab_size=201088, hidden_size=2880, num_layers=36,
        first_k_dense=0, moe_intermediate_size=2880, n_routed_experts=128, n_shared_experts=0,
        num_experts_per_tok=4, scoring_func="softmax", num_heads=64, num_kv_heads=8, head_dim=64,
        sliding_window=128, attention_sinks=True, activation="swiglu_clamped",
        rope_theta=150000.0, rope_interleaved=False, rope_scaling_factor=32.0, quant="mxfp4",
        quant_block=32)


def minimax_m25() -> ModelConfig:
    return ModelConfig(
        name="minimax-m2.5", family="minimax", vocab_size=200064, hidden_size=3072, num_layers=62,
        first_k_dense=0, moe_intermediate_size=1536, n_routed_experts=256, n_shared_experts=0,
        num_experts_per_tok=8, num_heads=48, num_kv_heads=8, head_dim=128, rope_interleaved=False,
        quant="fp8_block")


_PRESETS = {
    "tiny-deepseek-v3": tiny_deepseek_v3,
    "tiny-glm5": tiny_glm5,
    "tiny-kimi-k3": tiny_kimi_k3,
    "tiny-kimi-linear": tiny_kimi_linear,
    "tiny-kimi-k3.1": tiny_kimi_k31,
    "kimi-k3.1": kimi_k31,
    "kimi-k3-kda": kimi_k3_kda,
    "kimi-linear-48b": kimi_linear_48b,
    "tiny-gpt-oss": tiny_gpt_oss,
    "tiny-gpt-oss-64": tiny_gpt_oss_64,
    "tiny-minimax": tiny_minimax,
    "tiny-deepseek-v2": tiny_deepseek_v2,
    "tiny-mixtral": tiny_mixtral,
    "tiny-qwen2-moe": tiny_qwen2_moe,
    "tiny-deepseek-v4": tiny_deepseek_v4,
    "deepseek-v4-flash": deepseek_v4_flash,
    "deepseek-v4-pro": deepseek_v4_pro,
    "deepseek-v2": deepseek_v2_236b,
    "mixtral-8x7b": mixtral_8x7b,
    "mixtral-8x22b": mixtral_8x22b,
    "qwen2-57b-a14b": qwen2_57b_a14b,
    "qwen1.5-moe-a2.7b": qwen15_moe_a27b,
    "deepseek-v3-671b": deepseek_v3_671b,
    "deepseek-r1": deepseek_v3_671b,
    "glm-5.3-fp8": glm5_3,
    "kimi-k3": kimi_k3,
    "kimi-k2.5": kimi_k25,
    "gpt-oss-120b": gpt_oss_120b,
    "minimax-m2.5": minimax_m25,
}

# HF-style identity patterns -> preset (the reference matches on substrings of the model id,
# batchgen/config/model_registry.py:63-117).
_PATTERNS = [
    (r"deepseek[-_/]?(ai/)?.*(v3|r1)", "deepseek-v3-671b"),
    (r"deepseek[-_/]?(ai/)?.*v4[-_]?pro", "deepseek-v4-pro"),
    (r"deepseek[-_/]?(ai/)?.*v4", "deepseek-v4-flash"),
    (r"deepseek[-_/]?(ai/)?.*v2", "deepseek-v2"),
    (r"mixtral.*8x22b", "mixtral-8x22b"),
    (r"mixtral", "mixtral-8x7b"),
    (r"qwen1\.5[-_]?moe", "qwen1.5-moe-a2.7b"),
    (r"qwen2?[-_].*(moe|a14b)", "qwen2-57b-a14b"),
    (r"glm[-_]?5", "glm-5.3-fp8"),
    (r"kimi[-_]?linear", "kimi-linear-48b"),
    (r"kimi[-_]?k3\.1", "kimi-k3.1"),
    (r"kimi[-_]?k3[-_]?kda", "kimi-k3-kda"),
    (r"kimi[-_]?k3", "kimi-k3"),
    (r"kimi[-_]?k2", "kimi-k2.5"),
    (r"gpt[-_]?oss", "gpt-oss-120b"),
    (r"minimax", "minimax-m2.5"),
]


def list_models() -> List[str]:
    return sorted(_PRESETS)


def get_model_config(name: str, **overrides) -> ModelConfig:
    key = name.lower()
    if key not in _PRESETS:
        for pat, preset in _PATTERNS:
            if re.search(pat, key):
                key = preset
                break
        else:
            raise KeyError(f"unknown model {name!r}; known: {list_models()}")
    cfg = _PRESETS[key]()
    for k, v in overrides.items():
        if not hasattr(cfg, k):
            raise AttributeError(f"ModelConfig has no field {k!r}")
        setattr(cfg, k, v)
    return cfg


# ------------------------------------------------------------------ engine config
@dataclass
class EngineConfig:
    """Runtime knobs.  Names follow the reference's server flags where one exists
    (docs/server-flags.md; batchgen/server/server_args.py:168-285)."""
    page_size: int = 64
    kv_dtype: str = "bf16"                      # bf16 | fp8
    gpu_memory_frac: float = 0.9
    num_gpu_pages: int = 0                      # 0 = size from free memory
    host_kv_cache_size_gb: float = 0.0          # CPU-DRAM KV tier
    host_kv_chunk_size: int = 8192
    host_kv_watermark: int = 70
    initial_gpu_page_buffer: int = 32
    extension_gpu_page_buffer: int = 4
    decision_frequency_pages: int = 2
    max_prefill_tokens: int = 131072            # packed micro-batch token cap
    max_decode_batch: int = 512                 # rows per rank in decode
    max_state_slots: int = 0                    # sequences holding recurrent (KDA) state at once; 0 = max_decode_batch
    max_host_state_items: int = 0               # parked recurrent states in host memory; 0 = 4 x the device slots
    max_model_len: int = -1
    enable_cuda_graph: bool = True
    cuda_graph_max_bucket_size: int = 128
    cuda_graph_num_buckets: int = 16
    enable_prefix_cache: bool = False
    adaptive_chunk: bool = False
    adaptive_chunk_min: int = 1024              # bounds, smoothing and head-room of the adaptive host-KV chunk
    adaptive_chunk_max: int = 65536
    adaptive_chunk_ema_alpha: float = 0.1
    adaptive_chunk_multiplier: float = 1.5
    # parallel layout
    world_size: int = 1
    attn_tp_size: int = 1                       # TP degree of attention (1 = DP attention)
    ep_size: int = 1                            # expert parallel degree
    decode_attn_split: str = "heads"            # heads | requests: how a TP group divides the decode attention core
    moe_comm: str = "fused"                     # fused | nccl  (nccl = all_gather/reduce_scatter baseline)
    tp_comm: str = "fused"                      # fused | nccl
    expert_offload_ratio: float = 0.0           # fraction of local experts kept in host DRAM
    weight_ring_slots: int = 4
    seed: int = 0
    host_kv_backend: str = "native"       # "native": node-shared region + asynchronous movers (GPU); "torch": pinned tensor
    deferred_readback: bool = True      # with captured decode graphs: read a step's tokens while the next one runs
    device: str = "cpu"
    dtype: str = "fp32"                         # fp32 (CPU oracle) | bf16 (GPU)

    def validate(self) -> None:
        if self.page_size <= 0 or self.page_size & (self.page_size - 1):
            raise ValueError("page_size must be a power of two")
        if self.world_size % max(self.attn_tp_size, 1):
            raise ValueError("attn_tp_size must divide world_size")
        if self.ep_size not in (1, self.world_size):
            raise ValueError("ep_size must be 1 or world_size")
        if not 0.0 <= self.expert_offload_ratio <= 1.0:
            raise ValueError("expert_offload_ratio must be in [0, 1]")
        if self.decode_attn_split not in ("heads", "requests"):
            raise ValueError("decode_attn_split must be 'heads' or 'requests'")
        if self.kv_dtype not in ("bf16", "fp8", "fp32"):
            raise ValueError(f"unsupported kv dtype {self.kv_dtype}")

    @classmethod
    def from_json(cls, path: str) -> "EngineConfig":
        with open(path) as f:
            d = json.load(f)
        names = {f.name for f in dataclasses.fields(cls)}
        unknown = set(d) - names
        if unknown:
            raise ValueError(f"unknown engine config keys: {sorted(unknown)}")
        cfg = cls(**d)
        cfg.validate()
        return cfg
