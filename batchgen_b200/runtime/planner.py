"""Deployment planner: a bytes model of what one rank holds, and KV pool sizing from measured free memory.

The reference derives its batch configuration from fixed constants tuned for 96 GB GPUs
(batchgen/planner/base_planner.py:105-221: ``MAGIC_NUM // max_prompt_length``, 0.85 memory fraction); on a
180 GB part those constants are wrong, so this planner computes from bytes: weights per rank under the chosen
TP/EP layout, workspace for the largest prefill micro-batch, CUDA-graph capture memory, and gives the rest to
the KV page pool.  ``plan_deployment`` is pure (usable on CPU and in tests); ``size_kv_pool`` measures the live
device after the model is resident, like the reference's ``_init_gpu_kv_with_actual_size``
(batchgen/worker/kv_capacity_engine.py:455).  Machine profiles are keyed by family as in
batchgen/hardware/machine_family.py:40-115.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from ..config import EngineConfig, ModelConfig

GiB = 1 << 30


@dataclass(frozen=True)
class MachineProfile:
    name: str
    hbm_bytes: int
    hbm_gbs: float             # measured copy bandwidth
    bf16_tflops: float         # measured dense GEMM
    nvlink_gbs: float          # per direction per GPU
    sms: int
    host_dram_bytes: int


MACHINES: Dict[str, MachineProfile] = {
    "b200": MachineProfile("b200", 180 * GiB, 6450.0, 1434.0, 770.0, 148, 196 * GiB),
    "h200": MachineProfile("h200", 141 * GiB, 4000.0, 800.0, 400.0, 132, 1024 * GiB),
    "h20": MachineProfile("h20", 96 * GiB, 3400.0, 140.0, 400.0, 78, 1024 * GiB),
    "cpu": MachineProfile("cpu", 8 * GiB, 50.0, 1.0, 0.0, 1, 16 * GiB),
}


def machine_family(device_name: str) -> str:
    n = device_name.lower()
    for key in ("b200", "h200", "h20"):
        if key in n:
            return key
    return "cpu" if "cpu" in n else "b200"


@dataclass
class DeploymentPlan:
    weight_bytes: int
    expert_bytes: int
    workspace_bytes: int
    graph_bytes: int
    kv_bytes: int
    num_gpu_pages: int
    num_host_pages: int
    kv_token_capacity: int
    max_decode_batch: int
    fits: bool
    note: str = ""


def _quant_bytes(cfg: ModelConfig) -> float:
    return {"fp8_block": 1.0 + 4.0 / (128 * 128), "mxfp4": 0.5 + 1.0 / 32, "int4": 0.5 + 2.0 / 32, "none": 2.0}[cfg.quant]


def weight_bytes_per_rank(cfg: ModelConfig, tp: int, ep: int, sequence_parallel: bool = True,
                          expert_offload_ratio: float = 0.0) -> Tuple[int, int]:
    """-> (non-expert bytes, routed-expert bytes resident on the GPU) for one rank."""
    H = cfg.hidden_size
    qb = _quant_bytes(cfg)
    lin = 1.0 + 4.0 / (128 * 128) if cfg.quant != "none" else 2.0     # attention / dense linears are FP8 or bf16
    dense = 2 * cfg.vocab_size * H * 2 / (1 if sequence_parallel else tp)
    attn = 0.0
    if cfg.is_mla:
        attn += (cfg.q_lora_rank + cfg.kv_cache_dim) * H * lin
        attn += cfg.num_heads * cfg.qk_head_dim * cfg.q_lora_rank * lin / tp
        attn += cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim) * cfg.kv_lora_rank * 2 / tp
        attn += H * cfg.num_heads * cfg.v_head_dim * lin / tp
    else:
        attn += (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim * H * lin / tp
        attn += cfg.num_heads * cfg.head_dim * H * lin / tp
    experts = 0.0
    for l in range(cfg.num_layers):
        dense += attn
        if cfg.is_moe_layer(l):
            eh = cfg.expert_hidden
            experts += (cfg.n_routed_experts / ep) * 3 * eh * cfg.moe_intermediate_size * qb
            dense += cfg.n_shared_experts * 3 * H * cfg.moe_intermediate_size * lin / (1 if sequence_parallel else tp)
            dense += cfg.n_routed_experts * H * 4
        else:
            dense += 3 * H * cfg.intermediate_size * lin / tp
    return int(dense), int(experts * (1.0 - expert_offload_ratio))


def plan_deployment(cfg: ModelConfig, ecfg: EngineConfig, machine: MachineProfile, kv_dtype_bytes: int = 2) -> DeploymentPlan:
    tp = max(1, ecfg.attn_tp_size)
    ep = max(1, ecfg.ep_size)
    dense, experts = weight_bytes_per_rank(cfg, tp, ep, True, ecfg.expert_offload_ratio)
    # workspace of the largest prefill micro-batch: activations (bf16) of a few live tensors per token
    per_tok = cfg.hidden_size * 2 * 6 + cfg.num_heads // tp * (cfg.qk_head_dim + 2 * cfg.kv_cache_dim) * 2
    per_tok += cfg.num_experts_per_tok * (cfg.expert_hidden * 3 + cfg.moe_intermediate_size * 3) if cfg.n_routed_experts else 0
    workspace = int(min(ecfg.max_prefill_tokens, 32768) * per_tok * 1.25) + 2 * GiB
    graphs = int(0.5 * GiB + ecfg.cuda_graph_num_buckets * 64 * (1 << 20)) if ecfg.enable_cuda_graph else 0
    usable = int(machine.hbm_bytes * ecfg.gpu_memory_frac)
    kv = usable - dense - experts - workspace - graphs
    page_bytes = cfg.kv_bytes_per_token(kv_dtype_bytes) * ecfg.page_size
    pages = max(0, kv // page_bytes)
    if ecfg.num_gpu_pages:
        pages = min(pages, ecfg.num_gpu_pages) if pages else ecfg.num_gpu_pages
    host_pages = int(ecfg.host_kv_cache_size_gb * 1e9 // page_bytes)
    cap = pages * ecfg.page_size
    # decode rows: every live row needs its context plus the initial buffer; assume 4K contexts
    per_row = 4096 + ecfg.initial_gpu_page_buffer * ecfg.page_size
    rows = max(1, min(ecfg.max_decode_batch, cap // per_row if cap else 1))
    fits = kv > 0 and pages > 0
    note = "" if fits else (f"weights {dense + experts >> 30} GiB + workspace {workspace >> 30} GiB exceed "
                            f"{usable >> 30} GiB; raise --ep-offloading-ratio or the world size")
    return DeploymentPlan(dense, experts, workspace, graphs, max(kv, 0), int(pages), host_pages, int(cap), int(rows),
                          fits, note)


def state_pool_bytes(cfg: ModelConfig, ecfg: EngineConfig) -> int:
    """Device bytes of the per-sequence state pool (recurrent state of KDA layers, or the window rings and compressor
    windows of DeepSeek-V4): one slot per sequence that may be live at once."""
    slots = ecfg.max_state_slots or ecfg.max_decode_batch
    if cfg.is_v4:
        return slots * 4 * cfg.v4_state_floats_per_seq()
    return slots * cfg.kda_state_bytes_per_seq(max(ecfg.attn_tp_size, 1))


def size_kv_pool(cfg: ModelConfig, ecfg: EngineConfig, device: str, dtype) -> Tuple[int, int]:
    """Pages for the device pool and the host tier on the live machine (model already resident)."""
    import torch
    esz = torch.empty(0, dtype=dtype).element_size()
    page_bytes = cfg.kv_bytes_per_token(esz) * ecfg.page_size
    host_pages = int(ecfg.host_kv_cache_size_gb * 1e9 // page_bytes)
    if ecfg.num_gpu_pages:
        return ecfg.num_gpu_pages, host_pages
    if str(device).startswith("cuda"):
        free, total = torch.cuda.mem_get_info(torch.device(device))
        reserve = int(total * (1.0 - ecfg.gpu_memory_frac)) + 4 * GiB      # graphs + prefill workspace headroom
        if cfg.has_kda or cfg.is_v4:                                       # per-sequence state slots come out of the same memory
            reserve += state_pool_bytes(cfg, ecfg)
        pages = max(16, (free - reserve) // page_bytes)
        if ecfg.max_model_len > 0:
            pages = min(pages, ecfg.max_decode_batch * (-(-ecfg.max_model_len // ecfg.page_size) + 1))
        return int(pages), host_pages
    return 512, host_pages


def host_memory_preflight(cfg: ModelConfig, ecfg: EngineConfig, mem_total_bytes: int, world: int = 1) -> Optional[str]:
    """Refuse plans whose host-resident parts exceed MemTotal (reference: batchgen/host_memory_preflight.py).
    Returns None when fine, else the reason."""
    dense, experts_gpu = weight_bytes_per_rank(cfg, world, world, True, 0.0)
    host_experts = int(experts_gpu * ecfg.expert_offload_ratio) * world
    host_kv = int(ecfg.host_kv_cache_size_gb * 1e9) * world
    need = host_experts + host_kv + 8 * GiB
    if need > mem_total_bytes:
        return (f"host plan needs {need >> 30} GiB (offloaded experts {host_experts >> 30} GiB + host KV "
                f"{host_kv >> 30} GiB + 8 GiB runtime) but MemTotal is {mem_total_bytes >> 30} GiB")
    return None
