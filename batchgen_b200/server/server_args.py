"""Server flags: one dataclass, one argparse builder, cross-field validation.

Flag names follow the reference's (docs/server-flags.md; batchgen/server/server_args.py:168-322 dataclass,
:325 parser, :791 validation) so that launch scripts carry over.  Flags that only make sense for the
reference's multi-node / UCX / lane machinery are accepted where harmless and rejected with a clear
message where they would silently do nothing (``--nnodes > 1``).
"""
from __future__ import annotations

import argparse
import dataclasses
import os
from dataclasses import dataclass, field
from typing import List, Optional

from ..config import EngineConfig, list_models


@dataclass
class ServerArgs:
    # model / paths
    model: str = "tiny-deepseek-v3"         # preset name or a Hugging Face style id (config.get_model_config)
    cache_dir: str = ""                     # directory for derived files (converted shards, staged stores)
    converted_ckpt_dir: str = ""            # checkpoint in the converted format (ckpt.converter); empty = random weights
    tokenizer: str = "ids"                  # ids | bytes | a local tokenizer directory
    # topology
    world_size: int = 1                     # GPUs (ranks) of this server
    nnodes: int = 1                         # nodes of the deployment (one box: 1)
    node_rank: int = 0                      # this node's index
    dist_init_addr: str = "127.0.0.1:29600" # host:port of the ranks' rendezvous
    attn_tp_size: int = 0                       # 0 = world_size (TP attention), 1 = data-parallel attention
    device: str = "auto"                        # auto | cuda | cpu
    # memory
    host_kv_cache_size: float = 0.0             # GB of pinned host KV (overflow tier)
    kv_dtype: str = "bf16"                  # dtype of the paged KV (bf16)
    gpu_memory_frac: float = 0.9            # share of device memory the engine may use (KV pool = what the weights leave of it)
    num_gpu_pages: int = 0                  # KV pages on the device; 0 = sized from free memory
    max_model_len: int = -1                 # longest prompt + completion admitted; -1 = what the pool holds
    page_size: int = 64                     # tokens per KV page
    # scheduling
    initial_gpu_page_buffer: int = 32       # pages reserved ahead of a row when it starts decoding
    extension_gpu_page_buffer: int = 4      # pages added at every growth decision
    decision_frequency_pages: int = 2       # growth / hold decisions are taken every this many pages of progress
    host_kv_watermark: int = 70             # percent of free host KV above which parked rows are brought back eagerly
    host_kv_region: str = ""                   # set by the server: path of the node-shared host KV region's descriptor
    host_kv_chunk_size: int = 8192          # tokens of host KV reserved per parked row at a time
    adaptive_chunk: bool = False            # let the chunk follow the completed decode lengths (EMA)
    adaptive_chunk_min: int = 1024          # lower bound of the adaptive chunk, tokens
    adaptive_chunk_max: int = 65536         # upper bound of the adaptive chunk, tokens
    adaptive_chunk_ema_alpha: float = 0.1   # smoothing of the decode-length average
    adaptive_chunk_multiplier: float = 1.5  # head-room over the average
    max_decode_batch: int = 512             # decode rows per step
    max_prefill_tokens: int = 131072        # tokens of one packed prefill micro-batch; longer prompts are prefilled in pieces
    # offload
    enable_ep_with_offloading: bool = False # keep part of the routed experts in host memory and stream them
    ep_offloading_ratio: float = 0.0        # fraction of a rank's experts kept in host memory
    # graphs
    enable_cuda_graph: bool = True          # capture decode steps as CUDA graphs
    disable_cuda_graphs: bool = False       # overrides --enable-cuda-graph
    cuda_graph_max_bucket_size: int = 128   # largest captured batch bucket
    cuda_graph_num_buckets: int = 16        # number of batch buckets
    # prefix
    enable_prefix_cache: bool = False       # page-level prefix reuse (device cache + host coordinator, in-wave sharing, session frontiers)
    # comm
    moe_comm: str = "fused"                     # fused (in-kernel NVLink exchange) | nccl (collective baseline)
    fused_max_tokens: int = 16384               # largest step (prefill micro-batch) of the fused path; sizes its heap
    decode_attn_split: str = "auto"             # heads | requests (rows pinned to owner ranks inside the TP group) | auto:
                                                # requests on the fused multi-GPU path of an MLA model, heads otherwise
    # recurrent state (models with KDA layers)
    max_state_slots: int = 0                # sequences holding per-sequence state at once; 0 = max_decode_batch
    max_host_state_items: int = 0           # parked states in host memory; 0 = 4 x the device slots
    # output
    parse_thinking: bool = False            # split reasoning from content in chat responses
    parse_tool_call: bool = False           # parse the family's tool-call markup into tool_calls
    detokenization_include_special_tokens: bool = False  # keep special tokens in the returned text
    storage_path: str = "./batchgen_storage"   # directory of uploaded files, batches and outputs
    incremental_output_dir: str = ""        # append each finished request's item here as it completes (crash-resilient)
    # watchdogs
    watchdog_timeout: float = 600.0         # seconds without engine progress before the watchdog acts; 0 = off
    decode_step_timeout: float = 120.0      # seconds one decode step may take
    startup_timeout: float = 1800.0         # seconds the workers get to become ready
    startup_phase_timeout_scale: float = 1.0    # stretches the per-phase stall limits of the startup watchdog
    watchdog_test_stuck_time: float = 0.0       # fault injection (host side): worker sleeps this long once
    heartbeat_interval: float = 5.0             # seconds between worker heartbeats (counters, memory, parked rows)
    dp_migration: bool = True                   # hand parked rows of a loaded cohort to an idle one (--dp-size > 1)
    # logging
    log_dir: str = ""                       # JSONL event logs, flight recorder and stack dumps go here
    log_level: str = "info"                 # debug | info | warning | error
    # http
    weight_store_stage_dir: str = ""            # copy the converted checkpoint here first (local NVMe) and verify it
    shared_weight_store: bool = True            # load the converted checkpoint once into a node-shared region
    param_store_path: str = ""                  # set by the server: descriptor path of the shared weight region
    dp_size: int = 1                            # data-parallel cohorts: world_size / dp_size GPUs each, requests spread by sum of L^2
    query_book_mb: int = 64                     # node-shared token book (prompts + generated tokens), MiB
    instance_id: str = ""                       # stable name of this deployment (default: port<port>)
    run_mode: str = "exclusive"                 # "shared": several servers on the machine, a lane lease is mandatory
    runtime_root: str = ""                      # directory of the host / instance / run locks
    lane_manifest_fd: int = -1                  # inherited descriptor of the launcher's lane manifest
    lane_gpus: str = ""                         # leased GPU UUIDs (default: CUDA_VISIBLE_DEVICES)
    lane_lock_root: str = ""                    # directory of the per-GPU / per-port lane locks
    runtime_dir: str = ""                       # set by the server: this run's directory (workers take its run lock)
    run_id: str = ""                            # set by the server
    host: str = "127.0.0.1"                 # listen address
    port: int = 8000                        # listen port
    # capacity
    max_intake_capacity: int = 1_000_000    # requests the intake pool holds before new batches are refused
    scheduling_slots: int = 4096            # requests in flight on the workers at once
    # cluster
    cluster_fail_fast: bool = True          # a lost rank takes the cohort down at once (no hang on the next collective)
    seed: int = 0                           # seed of sampling and of random weights

    def engine_config(self) -> EngineConfig:
        tp = self.attn_tp_size or self.world_size
        return EngineConfig(
            page_size=self.page_size, kv_dtype=self.kv_dtype, gpu_memory_frac=self.gpu_memory_frac,
            num_gpu_pages=self.num_gpu_pages, host_kv_cache_size_gb=self.host_kv_cache_size,
            host_kv_chunk_size=self.host_kv_chunk_size, host_kv_watermark=self.host_kv_watermark,
            initial_gpu_page_buffer=self.initial_gpu_page_buffer,
            extension_gpu_page_buffer=self.extension_gpu_page_buffer,
            decision_frequency_pages=self.decision_frequency_pages, max_prefill_tokens=self.max_prefill_tokens,
            max_decode_batch=self.max_decode_batch, max_model_len=self.max_model_len,
            enable_cuda_graph=self.enable_cuda_graph and not self.disable_cuda_graphs,
            cuda_graph_max_bucket_size=self.cuda_graph_max_bucket_size,
            cuda_graph_num_buckets=self.cuda_graph_num_buckets, enable_prefix_cache=self.enable_prefix_cache,
            adaptive_chunk=self.adaptive_chunk, adaptive_chunk_min=self.adaptive_chunk_min,
            adaptive_chunk_max=self.adaptive_chunk_max, adaptive_chunk_ema_alpha=self.adaptive_chunk_ema_alpha,
            adaptive_chunk_multiplier=self.adaptive_chunk_multiplier, world_size=self.world_size, attn_tp_size=tp,
            ep_size=self.world_size, moe_comm=self.moe_comm, expert_offload_ratio=self.ep_offloading_ratio,
            decode_attn_split=("heads" if self.decode_attn_split == "auto" else self.decode_attn_split),
            max_state_slots=self.max_state_slots,
            max_host_state_items=self.max_host_state_items, seed=self.seed)


# Flags of the reference server that name the same setting differently here (reference flag -> field, converter).
REFERENCE_ALIASES = {
    "listen_ip": ("host", str), "listen_port": ("port", int), "max_pool_size": ("max_intake_capacity", int),
    "watchdog_heartbeat_interval": ("heartbeat_interval", float), "lane_lease_manifest_fd": ("lane_manifest_fd", int),
    "runtime_mode": ("run_mode", str), "runtime_identity": ("instance_id", str),
    "input_ids_pool_size_gb": ("query_book_mb", lambda v: max(1, int(float(v) * 1024))),
}
# Flags of the reference that have no counterpart to set: accepted (a launch script written for the reference keeps
# working) and reported once in the log with the reason.
REFERENCE_ACCEPTED = {
    "enable_host_kv_eviction": "eviction is always on with a host tier", "host_kv_eviction_watermark": "eviction is growth-driven",
    "enable_prepack": "prefill micro-batches are always packed", "enable_deepep": "the fused NVLink kernels are the exchange",
    "gpu_arch": "sm_100a only", "hf_cache_dir": "checkpoints are local directories", "pynccl_port_base": "no separate NCCL communicator",
    "pynccl_port_span": "no separate NCCL communicator", "replicated_weights": "weights live once per node in the shared store",
    "persistent_phase_instances": "one engine serves prefill and decode", "pre_dequantize_weights": "MXFP4 experts run on the W4A16 kernels",
    "glm5_disable_decode_host_kv_staging": "no staging path to disable", "save_result": "results are stored as batch output files",
    "prefix_cache_debug_stats": "prefix statistics are always in the heartbeat", "shared_prefix_admission": "shared prefixes are always charged once",
    "enable_decode_preemption": "rows are parked at page boundaries whenever the pool runs short", "fast_init": "weights are random unless a checkpoint is given",
    "enable_hugetlbfs": "the weight store asks for huge pages itself", "distributed_weight_config": "one node: the weight daemon is not started",
    "restart_control_addr": "one node: the restart coordinator uses the rendezvous address",
}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("batchgen_b200 server", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    compat = p.add_argument_group("flags of the reference server (aliases and accepted no-ops)")
    for name, (field, conv) in REFERENCE_ALIASES.items():
        compat.add_argument("--" + name.replace("_", "-"), dest=field, type=conv, default=argparse.SUPPRESS,
                            help=f"same as --{field.replace('_', '-')}")
    for name, why in REFERENCE_ACCEPTED.items():
        compat.add_argument("--" + name.replace("_", "-"), dest="_accepted_" + name, nargs="?", const=True,
                            default=argparse.SUPPRESS, help=f"accepted, no effect: {why}")
    for f in dataclasses.fields(ServerArgs):
        flag = "--" + f.name.replace("_", "-")
        if f.type in ("bool", bool):
            p.add_argument(flag, action="store_true", default=f.default)
            if f.default:
                p.add_argument("--no-" + f.name.replace("_", "-"), dest=f.name, action="store_false")
        else:
            typ = {"int": int, "float": float, "str": str}.get(f.type if isinstance(f.type, str) else f.type.__name__, str)
            p.add_argument(flag, type=typ, default=f.default)
    return p


class ServerArgsError(ValueError):
    pass


def validate_server_args(a: ServerArgs) -> ServerArgs:
    if a.nnodes != 1 or a.node_rank != 0:
        raise ServerArgsError("this engine serves one NVSwitch node: --nnodes must be 1 (the reference's multi-node "
                              "restart coordinator and UCX weight store have no counterpart here)")
    if a.world_size < 1 or a.world_size > 8 or a.world_size & (a.world_size - 1):
        raise ServerArgsError("--world-size must be 1, 2, 4 or 8")
    if a.dp_size < 1 or a.world_size % a.dp_size:
        raise ServerArgsError("--dp-size must divide --world-size")
    if a.attn_tp_size not in (0, 1, a.world_size):
        raise ServerArgsError("--attn-tp-size must be 1 (DP attention) or the world size")
    if not 0.1 <= a.gpu_memory_frac <= 0.98:
        raise ServerArgsError("--gpu-memory-frac must be within [0.1, 0.98]")
    if a.host_kv_cache_size < 0:
        raise ServerArgsError("--host-kv-cache-size must be >= 0 GB")
    if a.kv_dtype not in ("bf16", "fp8", "fp32"):
        raise ServerArgsError("--kv-dtype must be bf16, fp8 or fp32")
    if a.page_size <= 0 or a.page_size & (a.page_size - 1):
        raise ServerArgsError("--page-size must be a power of two")
    if a.extension_gpu_page_buffer < a.decision_frequency_pages:
        raise ServerArgsError("--extension-gpu-page-buffer must cover a decision interval "
                              "(>= --decision-frequency-pages)")
    if not 0 <= a.host_kv_watermark <= 100:
        raise ServerArgsError("--host-kv-watermark is a percentage")
    if a.enable_ep_with_offloading and not 0 < a.ep_offloading_ratio <= 1:
        raise ServerArgsError("--enable-ep-with-offloading needs --ep-offloading-ratio in (0, 1]")
    if not a.enable_ep_with_offloading and a.ep_offloading_ratio:
        raise ServerArgsError("--ep-offloading-ratio needs --enable-ep-with-offloading")
    if a.moe_comm not in ("fused", "nccl"):
        raise ServerArgsError("--moe-comm must be fused or nccl")
    if a.fused_max_tokens < 8 * a.world_size:
        raise ServerArgsError("--fused-max-tokens must hold at least 8 rows per rank")
    if a.cuda_graph_max_bucket_size <= 0 or a.cuda_graph_num_buckets <= 0:
        raise ServerArgsError("CUDA graph bucket settings must be positive")
    if a.log_level not in ("debug", "info", "warning", "error"):
        raise ServerArgsError("--log-level must be debug, info, warning or error")
    if a.max_intake_capacity <= 0 or a.scheduling_slots <= 0:
        raise ServerArgsError("capacities must be positive")
    if a.converted_ckpt_dir and not os.path.isdir(a.converted_ckpt_dir):
        raise ServerArgsError(f"--converted-ckpt-dir {a.converted_ckpt_dir} is not a directory")
    try:
        from ..config import get_model_config
        get_model_config(a.model)
    except KeyError:
        raise ServerArgsError(f"unknown --model {a.model!r}; known: {list_models()}")
    return a


def prepare_server_args(argv: Optional[List[str]] = None) -> ServerArgs:
    ns = vars(build_parser().parse_args(argv))
    accepted = sorted(k[len("_accepted_"):] for k in ns if k.startswith("_accepted_"))
    args = validate_server_args(ServerArgs(**{k: v for k, v in ns.items() if not k.startswith("_accepted_")}))
    args.accepted_reference_flags = accepted             # launch.py logs them with the reason each has no effect
    return args


def flags_markdown() -> str:
    """The flag reference (``docs/server-flags.md``): one table per section of ``ServerArgs``, read from this file's
    own field comments.  ``python -m batchgen_b200.server.server_args > docs/server-flags.md`` regenerates it."""
    import re
    rows, section = [], ""
    for line in open(__file__, encoding="utf-8").read().split("@dataclass\nclass ServerArgs:")[1].split("def engine_config")[0].splitlines():
        m = re.match(r"\s{4}# (.+)$", line)
        if m:
            section = m.group(1).strip()
            continue
        m = re.match(r"\s{4}([a-z_0-9]+):\s*([A-Za-z\[\], \.]+?)\s*=\s*(.+?)(?:\s+#\s*(.*))?$", line)
        if m:
            rows.append((section, m.group(1), m.group(2), m.group(3).strip(), (m.group(4) or "").strip()))
    out = ["# Server flags", "",
           "`python -m batchgen_b200.server.launch [flags]`.  Every field of `server/server_args.py::ServerArgs` is a flag",
           "(`--field-name`; boolean fields that default to on also take `--no-field-name`).  This page is generated from",
           "that dataclass: `python -m batchgen_b200.server.server_args > docs/server-flags.md`."]
    current = None
    for sec, name, typ, default, note in rows:
        if sec != current:
            out += ["", f"## {sec}", "", "| flag | type | default | meaning |", "|---|---|---|---|"]
            current = sec
        out.append(f"| `--{name.replace('_', '-')}` | {typ} | `{default}` | {note.replace('|', 'or')} |")
    out += ["", "## Flags of the reference server", "",
            "A launch script written for the reference keeps working: these names are understood as well.", "",
            "| reference flag | here |", "|---|---|"]
    for k, (field, _) in REFERENCE_ALIASES.items():
        extra = " (GB are converted to MiB)" if k == "input_ids_pool_size_gb" else ""
        out.append(f"| `--{k.replace('_', '-')}` | same as `--{field.replace('_', '-')}`{extra} |")
    for k, why in REFERENCE_ACCEPTED.items():
        out.append(f"| `--{k.replace('_', '-')}` | accepted, no effect: {why} |")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    print(flags_markdown(), end="")
