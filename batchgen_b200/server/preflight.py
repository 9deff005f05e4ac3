"""Fail-closed preflights run before the server binds its port.

* launch readiness — storage and checkpoint paths reachable and writable, the HTTP port free;
* runtime preflight — the dependency contract of the chosen model: the in-tree kernel library exists (and was
  built for sm_100a) whenever a GPU will be used, the GPU is a compute-capability 10.x part, torch has the
  collectives backend the world size needs;
* host-memory preflight — offloaded experts + host KV fit ``MemTotal``.

Reference parity: batchgen/launch_readiness.py, batchgen/runtime_preflight.py:160-337,
batchgen/host_memory_preflight.py.
"""
from __future__ import annotations

import os
import socket
from typing import List


class PreflightError(RuntimeError):
    pass


def mem_total_bytes() -> int:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return 0


def launch_readiness(args) -> List[str]:
    out = []
    os.makedirs(args.storage_path, exist_ok=True)
    probe = os.path.join(args.storage_path, ".write_probe")
    try:
        with open(probe, "w") as f:
            f.write("ok")
        os.remove(probe)
    except OSError as e:
        raise PreflightError(f"--storage-path {args.storage_path} is not writable: {e}")
    out.append(f"storage path {args.storage_path} writable")
    if args.converted_ckpt_dir:
        if not any(n.endswith(".bin") for n in os.listdir(args.converted_ckpt_dir)):
            raise PreflightError(f"--converted-ckpt-dir {args.converted_ckpt_dir} holds no converted .bin shards")
        out.append("converted checkpoint present")
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((args.host, args.port))
        except OSError as e:
            raise PreflightError(f"cannot bind {args.host}:{args.port}: {e}")
    out.append(f"port {args.port} free")
    return out


def runtime_preflight(args) -> List[str]:
    import torch
    out = []
    want_gpu = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    if want_gpu:
        from ..ops import _ext
        if not _ext.available():
            raise PreflightError("the sm_100a kernel library is missing: run `python -m batchgen_b200.build`")
        if torch.cuda.device_count() < args.world_size:
            raise PreflightError(f"--world-size {args.world_size} but only {torch.cuda.device_count()} GPU(s) visible")
        major, minor = torch.cuda.get_device_capability(0)
        if major != 10:
            raise PreflightError(f"the kernels are built for sm_100a only; device 0 is sm_{major}{minor}")
        out.append(f"kernel library present, {torch.cuda.device_count()} x sm_{major}{minor}")
        if args.world_size > 1 and not torch.distributed.is_nccl_available():
            raise PreflightError("torch was built without NCCL")
        from ..config import get_model_config
        out += model_contract(get_model_config(args.model), args.world_size // max(getattr(args, "dp_size", 1), 1), True,
                              getattr(args, "moe_comm", "nccl"))
    else:
        from ..config import get_model_config
        out += model_contract(get_model_config(args.model), args.world_size // max(getattr(args, "dp_size", 1), 1), False)
        if args.world_size > 1 and not torch.distributed.is_gloo_available():
            raise PreflightError("torch was built without gloo")
        out.append("CPU execution (fp32 reference path)")
    return out


def model_contract(cfg, world: int, on_gpu: bool, moe_comm: str = "nccl") -> List[str]:
    """The dependency contract of one model on this engine: which geometries the hand-written kernels tile.  On a GPU
    a model outside the contract would raise ``KernelError`` at its first step (no silent library fallback); here it
    is refused before the workers start, with every violated rule in the message.  Returns notes for the log."""
    notes, bad = [], []
    if world > 1:
        if cfg.num_heads % world:
            bad.append(f"{cfg.num_heads} attention heads do not divide over {world} ranks")
        if cfg.n_routed_experts and cfg.n_routed_experts % world:
            bad.append(f"{cfg.n_routed_experts} routed experts do not divide over {world} ranks")
    if not on_gpu:
        if bad:
            raise PreflightError("model contract: " + "; ".join(bad))
        return ["fp32 reference path: no kernel geometry rules apply"]
    heads = cfg.num_heads // max(world, 1)
    if cfg.hidden_size % 128:
        bad.append(f"hidden_size {cfg.hidden_size} is not a multiple of 128 (1 x 128 FP8 activation groups)")
    if cfg.quant in ("fp8_block", "mxfp4", "int4"):
        for name, v in (("moe_intermediate_size", cfg.moe_intermediate_size), ("intermediate_size", cfg.intermediate_size)):
            if v and v % 128:
                bad.append(f"{name} {v} is not a multiple of 128")
    elif cfg.quant not in ("none",):
        bad.append(f"quant {cfg.quant!r} has no kernel")
    if cfg.is_v4:
        k_o = cfg.num_heads * cfg.head_dim // max(cfg.o_groups, 1)
        for name, v in (("q_lora_rank", cfg.q_lora_rank), ("head_dim", cfg.head_dim),
                        ("heads * head_dim / o_groups", k_o), ("o_groups * o_lora_rank", cfg.o_groups * cfg.o_lora_rank)):
            if v % 64:
                bad.append(f"{name} {v} is not a multiple of 64 (K of the projection GEMMs)")
        if world > 1:
            notes.append("DeepSeek-V4: attention replicated per engine, experts expert-parallel; use --dp-size for "
                         "data-parallel cohorts")
        notes.append("DeepSeek-V4: decode attention core on the MLA decode kernel (512-wide heads), prefill core and compressor as torch ops; projections, "
                     "router and experts run on the kernels")
    elif cfg.is_mla:
        if cfg.kv_lora_rank != 512 or cfg.qk_rope_head_dim != 64:
            bad.append(f"MLA kernels need kv_lora_rank 512 + rope 64 (got {cfg.kv_lora_rank} + {cfg.qk_rope_head_dim})")
        if cfg.qk_nope_head_dim % 64:
            bad.append(f"qk_nope_head_dim {cfg.qk_nope_head_dim} is not a multiple of 64 (absorb GEMM)")
        if heads % 8:
            bad.append(f"{heads} heads per rank: the MLA kernels tile multiples of 8 (64 for the persistent decode kernel)")
        notes.append("MLA decode: persistent kernel" if heads % 64 == 0 else "MLA decode: split-KV kernel (heads per rank not a multiple of 64)")
    else:
        if cfg.head_dim not in (64, 128):
            bad.append(f"GQA head_dim {cfg.head_dim}: the paged decode kernel covers 64 and 128")
        notes.append("GQA prefill runs the reference path (no prefill kernel)")
    if cfg.has_dsa and (cfg.index_n_heads != 32 or cfg.index_head_dim != 128):
        bad.append(f"DSA indexer kernels need 32 heads x 128 (got {cfg.index_n_heads} x {cfg.index_head_dim})")
    if cfg.has_kda and cfg.kda_head_dim not in (64, 128):
        bad.append(f"KDA head_dim {cfg.kda_head_dim}: the kernel covers 64 and 128")
    if world > 1 and moe_comm == "fused":
        from ..models.transformer import Transformer
        why = ("DeepSeek-V4 attention is replicated inside an engine" if cfg.is_v4
               else Transformer.supports_sequence_parallel(cfg))
        notes.append("fused NVLink path" if why is None else f"NCCL layout instead of the fused path: {why}")
    if bad:
        raise PreflightError("model contract: " + "; ".join(bad))
    return notes or ["model geometry within the kernels' contract"]


def host_memory(args) -> List[str]:
    from ..config import get_model_config
    from ..runtime.planner import host_memory_preflight
    total = mem_total_bytes()
    if total == 0:
        return ["MemTotal unknown: host-memory check skipped"]
    why = host_memory_preflight(get_model_config(args.model), args.engine_config(), total, args.world_size)
    if why:
        raise PreflightError(why)
    return [f"host plan fits MemTotal {total >> 30} GiB"]


def _gpu_name() -> str:
    """Name of GPU 0 through NVML (no CUDA context is created in the server process); "b200" when NVML is not there."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            name = pynvml.nvmlDeviceGetName(pynvml.nvmlDeviceGetHandleByIndex(0))
        finally:
            pynvml.nvmlShutdown()
        return name.decode() if isinstance(name, bytes) else str(name)
    except Exception:  # noqa: BLE001
        return "b200"


def deployment_plan(args) -> List[str]:
    """The per-GPU memory plan of the model on this machine (weights, experts, workspace, what is left for KV), as
    one log line; on a GPU a plan that leaves nothing for KV is refused unless the pool size is given explicitly."""
    from ..config import get_model_config
    from ..runtime import planner
    try:
        import torch
        on_gpu = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    except Exception:  # noqa: BLE001 - no torch / no driver: plan for the CPU profile
        on_gpu = False
    name = _gpu_name() if on_gpu else "cpu"
    if not on_gpu:
        return ["deployment plan: CPU run, sized by --num-gpu-pages"]
    cfg = get_model_config(args.model)
    world = max(1, args.world_size // max(1, getattr(args, "dp_size", 1)))
    machine = planner.MACHINES[planner.machine_family(name)]
    ecfg = args.engine_config()
    ecfg.world_size = ecfg.attn_tp_size = ecfg.ep_size = world
    plan = planner.plan_deployment(cfg, ecfg, machine)
    gib = lambda b: f"{b / 2 ** 30:.1f} GiB"
    line = (f"deployment plan ({machine.name}, {world} GPUs per cohort): dense {gib(plan.weight_bytes)}, experts "
            f"{gib(plan.expert_bytes)}, workspace + graphs {gib(plan.workspace_bytes + plan.graph_bytes)}, KV {gib(plan.kv_bytes)} "
            f"= {plan.kv_token_capacity} tokens per GPU")
    if not plan.fits and not args.num_gpu_pages:
        raise PreflightError(f"{line}; {plan.note}")
    return [line if plan.fits else f"{line}; {plan.note} (continuing: --num-gpu-pages is set)"]


def run_all_preflights(args) -> List[str]:
    return launch_readiness(args) + runtime_preflight(args) + host_memory(args) + deployment_plan(args)
