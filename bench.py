#!/usr/bin/env python
"""Headline benchmark: decode throughput (and prefill throughput / projected batch completion time)
of the DeepSeek-V3/R1-671B architecture, block-scaled FP8, tensor-parallel attention + expert-parallel
MoE over N GPUs of one node, on the 512-request workload (prompts U[512, 4096], 1,024 forced decode
tokens) with synthetic token ids and random-init weights.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)

A *step* is one decode step of the whole decode batch through all 61 layers, sampling included.
``value`` = decode tokens/s of the job (rows * K / time of K steps, device-timed with CUDA events,
max over ranks): the whole-step CUDA graph replayed on fixed device-resident inputs.

The ``e2e`` block times K real decode steps through the engine's public API (``Engine.decode_steps``): the
same sequences are registered with the engine (``Engine.adopt_sequence``: their synthetic KV already sits in
its page pool), and every step goes through the scheduler's admission, the per-step input staging from pinned
host memory (host->device copies of ids / positions / slots / lengths / block table), the graph replay, the
sampler with per-row parameters, the token all-gather on multi-GPU jobs and the device->host read of the
sampled tokens that the host needs to append them and to test for completion.

``--bct`` runs the whole 512-request workload (prompts U[512, 4096], 1,024 forced tokens) through the offline
batch API (``runtime.batch_api.run_batch``) on the same engine and adds the measured batch completion time and
the engine-reported prefill / decode rates to the line (key ``bct``); ``--bct-requests`` / ``--bct-tokens``
shrink it for quick runs (then marked ``"full": false``).

``--workload distinct64k | grouped64k`` (with ``--model glm-5.3-fp8``) runs the long-context workloads of the
sparse-attention (DSA) model through the same batch API instead of the decode-step benchmark: ``--requests`` prompts
of ``--ctx-tokens`` distinct tokens each, or ``--requests / 8`` shared prefixes with eight 64-token suffixes each,
``--bct-tokens`` forced decode tokens; the line reports the measured completion time and the engine's prefill and
decode rates.

Where the FP8 expert weights of the rank exceed what HBM can hold next to the KV pool (N < 8),
layers share physical expert storage in a cycle of ``distinct_expert_sets`` sets: every layer still
streams its full expert bytes from HBM (a set is far larger than L2) and executes every FLOP.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm(args) -> int:
    """The unmodified reference from baseline/_ref through its own public API."""
    why = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import importlib
        importlib.import_module("batchgen.native_loader")
        importlib.import_module("batchgen.core_engine")
    except Exception as e:  # noqa: BLE001
        why = f"reference does not import on this image: {type(e).__name__}: {str(e)[:160]}"
    if why is None:
        why = ("reference imports but its Blackwell path needs FlashMLA/DeepGEMM/UCX libraries that are not "
               "installed and cannot be fetched offline")
    if int(os.environ.get("RANK", "0")) == 0:          # one line for the whole job, whatever the launcher started
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")}))
    return 0


def run_bct(eng, cfg, args, rank, world, barrier):
    """The BASELINE workload through the offline batch API on the engine: wall time from the first request
    handed over to the last completion, plus the engine's own prefill / decode rates (the reference prints the
    same two at batchgen/batchgen_worker.py:6558-6578)."""
    import random as _random
    import time as _time

    from batchgen_b200.runtime import batch_api
    from batchgen_b200.runtime.engine import EngineStats
    from batchgen_b200.runtime.tokenization import get_tokenizer
    for s in list(eng.seqs.values()):                      # rows of the step benchmark leave first
        if s.status.name != "COMPLETED":
            eng._complete(s, "length")
    eng.seqs.clear()
    eng.stats = EngineStats()
    rng = _random.Random(99)
    reqs = []
    for i in range(args.bct_requests):
        n = rng.randint(512, 4096)
        ids = [rng.randrange(2, cfg.vocab_size) for _ in range(n)]
        reqs.append(batch_api.BatchRequest(f"r{i}", "/v1/completions",
                                           {"prompt": ids, "max_tokens": args.bct_tokens, "temperature": 0,
                                            "ignore_eos": True}))
    tok = get_tokenizer("ids", cfg.vocab_size)
    barrier()
    t0 = _time.perf_counter()
    items = batch_api.run_batch(eng, reqs, tok, batch_api.BatchOptions(endpoint="/v1/completions"))
    barrier()
    wall = _time.perf_counter() - t0
    ok = sum(1 for it in items if it["error"] is None)
    st = eng.stats.summary()
    return {"bct_s": wall, "requests": args.bct_requests, "completed": ok, "forced_tokens": args.bct_tokens,
            "full": args.bct_requests == 512 and args.bct_tokens == 1024,
            "prefill_tok_per_s": st["prefill_tok_per_s"], "decode_tok_per_s": st["decode_tok_per_s"],
            "prefill_tokens": st["prefill_tokens"], "decode_tokens": st["decode_tokens"],
            "prefill_waves": st["prefill_waves"], "decode_steps": st["decode_steps"], "holds": st["holds"],
            "evictions": st["evictions"], "api": "runtime.batch_api.run_batch on Engine"}


def run_longctx(args) -> int:
    """Long-context workloads (BASELINE configs 3 and 4) through Engine + batch API: chunked prefill of
    ``--ctx-tokens``-token prompts (8,192-token pieces; the DSA indexer scores every earlier key for each query and
    the attention reads the 2,048 selected rows), in-wave prefix sharing for the grouped form, then sparse decode."""
    import torch
    import torch.distributed as dist

    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.weights import ParallelLayout
    from batchgen_b200.ops import _ext
    from batchgen_b200.runtime import batch_api
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.kv_cache import host_page_bytes
    from batchgen_b200.runtime.tokenization import get_tokenizer
    from batchgen_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from batchgen_b200.parallel import make_comm
        comm = make_comm("nccl", None)                  # DSA layers run the tensor-parallel layout over NCCL
    _ext.lib()
    cfg = get_model_config(args.model)
    if args.layers:
        cfg.num_layers = args.layers
        cfg.indexer_full_layers = tuple(l for l in cfg.indexer_full_layers if l < args.layers)
        cfg.compress_ratios = tuple(cfg.compress_ratios[: args.layers])
    if args.experts:
        cfg.n_routed_experts = args.experts
    page, L, N, R = 64, args.ctx_tokens, args.bct_tokens, args.requests
    grouped = args.workload == "grouped64k"
    groups = max(1, R // 8) if grouped else R
    rng = random.Random(4321)
    if grouped:
        prefixes = [[rng.randrange(2, cfg.vocab_size) for _ in range(L - 64)] for _ in range(groups)]
        prompts = [prefixes[i // 8] + [rng.randrange(2, cfg.vocab_size) for _ in range(64)] for i in range(groups * 8)]
    else:
        prompts = [[rng.randrange(2, cfg.vocab_size) for _ in range(L)] for _ in range(R)]
    R = len(prompts)
    per_req = (L + N) // page + 3
    total_pages = (groups * (L // page) + R * (N // page + 4) + 16) if grouped else (R * per_req + 16)
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    n_moe = cfg.num_layers - cfg.first_k_dense
    expert_bytes_layer = (cfg.n_routed_experts // world) * 3 * cfg.moe_intermediate_size * cfg.hidden_size
    kv_bytes = total_pages * host_page_bytes(cfg, page)
    free_b, _ = torch.cuda.mem_get_info(dev)
    other = 30e9 / world + 16e9                               # attention / dense / shared / embeddings + workspace
    budget = free_b * 0.94 - kv_bytes - other
    if budget < expert_bytes_layer:
        raise SystemExit(f"{R} requests of {L} tokens need {kv_bytes / 1e9:.0f} GB of KV: too many for this GPU")
    sets = int(max(1, min(n_moe, budget // expert_bytes_layer)))
    alias = 0 if sets >= n_moe else sets
    t0 = time.time()
    model = build_model(cfg, device=dev, dtype="bf16", seed=0, layout=layout, comm=comm,
                        max_positions=L + N + 2 * page, alias_experts_every=alias, gen_device=dev)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    ecfg = EngineConfig(page_size=page, max_decode_batch=max(R, 8), max_prefill_tokens=args.prefill_tokens,
                        enable_cuda_graph=False, enable_prefix_cache=not cfg.is_v4, initial_gpu_page_buffer=N // page + 2,
                        extension_gpu_page_buffer=2, decision_frequency_pages=2, world_size=world,
                        attn_tp_size=world, ep_size=world, device=str(dev), dtype="bf16", moe_comm="nccl")
    eng = Engine(model, ecfg, num_gpu_pages=total_pages)
    graph_note = "eager"
    if not args.no_graph and world == 1:
        # the decode step (indexer, top-k, gather, sparse attention, experts) as one CUDA graph per batch bucket
        from batchgen_b200.runtime.graphs import DecodeGraphRunner
        try:
            eng.graph_runner = DecodeGraphRunner(model, eng.kv, max_batch=max(R, 8), max_pages_per_seq=per_req,
                                                 num_buckets=2, max_bucket=max(R, 8))
            eng.graph_runner.capture_all()
            graph_note = "cuda graph"
        except Exception as exc:                           # noqa: BLE001 - reported in the line, eager decode instead
            eng.graph_runner = None
            graph_note = f"eager (capture failed: {type(exc).__name__}: {str(exc)[:120]})"
            torch.cuda.synchronize()
    reqs = [batch_api.BatchRequest(f"r{i}", "/v1/completions",
                                   {"prompt": p, "max_tokens": N, "temperature": 0, "ignore_eos": True})
            for i, p in enumerate(prompts)]
    tok = get_tokenizer("ids", cfg.vocab_size)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    l0 = _ext.LAUNCHES["count"]
    barrier()
    t0 = time.perf_counter()
    items = batch_api.run_batch(eng, reqs, tok, batch_api.BatchOptions(endpoint="/v1/completions"))
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if sampler is not None else None
    _ext.check_status()
    st = eng.stats.summary()
    if rank == 0:
        ok = sum(1 for it in items if it["error"] is None)
        full = (args.model == "glm-5.3-fp8" and L == 65536 and N == 4096 and not args.layers
                and R == (512 if grouped else 312))
        print(json.dumps({
            "metric": f"batch completion time ({cfg.name}, {args.workload})", "value": wall, "unit": "s",
            "n_gpus": world, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "impl": "ours",
            "dtype": "fp8(e4m3 block-scaled weights+activations, e4m3 index keys)/bf16", "data": "synthetic",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "workload": args.workload, "requests": R,
                       "completed": ok, "ctx_tokens": L, "forced_tokens": N, "prefix_groups": groups if grouped else 0,
                       "parallelism": f"tp{world}+ep{world}", "comm": "nccl" if world > 1 else "none",
                       "prefill_piece_tokens": args.prefill_tokens, "index_topk": cfg.index_topk, "decode": graph_note,
                       "distinct_expert_sets": sets, "full_size_workload": full,
                       "valid": not args.layers and not args.experts, "experts": cfg.n_routed_experts,
                       "api": "runtime.batch_api.run_batch on Engine", "build_seconds": round(build_s, 1)},
            "prefill_tok_per_s": st["prefill_tok_per_s"], "decode_tok_per_s": st["decode_tok_per_s"],
            "prefill_tokens": st["prefill_tokens"], "shared_prefix_tokens": st["shared_prefix_tokens"],
            "prefill_chunks": st["prefill_chunks"], "prefill_seconds": st["prefill_seconds"],
            "decode_tokens": st["decode_tokens"], "decode_seconds": st["decode_seconds"],
            "decode_steps": st["decode_steps"], "clocks": clocks, "gpu_launches": _ext.LAUNCHES["count"] - l0}))
    sys.stdout.flush()
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_streamed(args) -> int:
    """Host-resident experts (BASELINE config 5 shape at a size one box holds): a Kimi-K3-shaped model whose routed
    experts stay in pinned host memory and flow through the native weight ring, one pass per forward.  The step is
    bound by the host-to-device copy, so the line reports the ring's achieved copy rate next to a plain pinned copy
    measured in the same process."""
    import random

    import torch

    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.ops import _ext
    from batchgen_b200.runtime import batch_api
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.tokenization import get_tokenizer
    from batchgen_b200.utils.clocks import ClockSampler

    assert args.gpus == 1, "the streamed workload runs on one GPU"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _ext.lib()
    model_name = args.model if args.model != "deepseek-v3-671b" else "kimi-k3"
    cfg = get_model_config(model_name)
    full_layers, full_experts = cfg.num_layers, cfg.n_routed_experts
    cfg.num_layers = args.layers or 8
    cfg.n_routed_experts = args.experts or 64
    R, L, N, page = args.requests if args.requests > 2 else 64, 256, args.bct_tokens if args.bct_tokens != 1024 else 32, 64
    # anchor: a plain pinned-host -> device copy of 1 GiB
    src = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
    dst = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        dst.copy_(src, non_blocking=True)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(4):
        dst.copy_(src, non_blocking=True)
    ev1.record()
    torch.cuda.synchronize()
    anchor_gbs = 4 * (1 << 30) / (ev0.elapsed_time(ev1) * 1e-3) / 1e9
    del src, dst
    t0 = time.time()
    model = build_model(cfg, device=dev, dtype="bf16", seed=0, max_positions=L + N + 2 * page, gen_device=dev,
                        stream_experts=True, ring_slots=3)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    per_req = (L + N) // page + 3
    ecfg = EngineConfig(page_size=page, max_decode_batch=R, enable_cuda_graph=False, initial_gpu_page_buffer=N // page + 2,
                        extension_gpu_page_buffer=2, decision_frequency_pages=2, device=str(dev), dtype="bf16")
    eng = Engine(model, ecfg, num_gpu_pages=R * per_req + 16)
    rng = random.Random(99)
    reqs = [batch_api.BatchRequest(f"r{i}", "/v1/completions",
                                   {"prompt": [rng.randrange(2, cfg.vocab_size) for _ in range(L)], "max_tokens": N,
                                    "temperature": 0, "ignore_eos": True}) for i in range(R)]
    tok = get_tokenizer("ids", cfg.vocab_size)
    sampler = ClockSampler(0).start()
    l0 = _ext.LAUNCHES["count"]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    items = batch_api.run_batch(eng, reqs, tok, batch_api.BatchOptions(endpoint="/v1/completions"))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    _ext.check_status()
    st = eng.stats.summary()
    ring = model.streamer.stats()
    passes = ring["bytes_copied"] / max(model.streamer.bytes_per_pass, 1)
    step_ms = 1e3 * st["decode_seconds"] / max(st["decode_steps"], 1)
    print(json.dumps({
        "metric": f"decode tokens/s with host-resident experts ({cfg.name} shape, reduced depth and expert count)",
        "value": st["decode_tok_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "vs_baseline": None,
        "impl": "ours", "dtype": "mxfp4 experts (W4A16) / bf16", "data": "synthetic",
        "config": {"model": cfg.name, "layers": cfg.num_layers, "of_layers": full_layers, "experts": cfg.n_routed_experts,
                   "of_experts": full_experts, "requests": R, "completed": sum(1 for it in items if it["error"] is None),
                   "prompt_tokens": L, "forced_tokens": N, "ring_slots": 3, "decode": "eager (host waits between layers)",
                   "valid": False, "note": "reduced size: the full model needs 1.4 TB of host memory",
                   "api": "runtime.batch_api.run_batch on Engine", "build_seconds": round(build_s, 1)},
        "wall_s": wall, "decode_ms_per_step": step_ms, "decode_steps": st["decode_steps"],
        "prefill_tok_per_s": st["prefill_tok_per_s"],
        "expert_bytes_per_pass": model.streamer.bytes_per_pass, "passes": passes,
        "step_h2d_gbs": model.streamer.bytes_per_pass / max(step_ms * 1e-3, 1e-9) / 1e9,
        "pinned_copy_gbs": anchor_gbs, "ring_stalls": ring["stalls"], "get_wait_ms": ring["get_wait_us"] / 1e3,
        "clocks": clocks, "gpu_launches": _ext.LAUNCHES["count"] - l0}))
    sys.stdout.flush()
    model.streamer.close()
    return 0


def compare_with_nccl(model, kv, d_ids, d_pos, d_slot, d_bt, d_len, rank, world, dist, n_layers=None):
    """Largest relative difference between one decode step over the fused kernels and the same step over NCCL
    collectives, on the same weights and inputs.  The baseline model shares every tensor with the fused one; only
    the tensors the sequence-parallel layout replicates are cut to their tensor-parallel shard.  Both runs use the
    first dense layers plus two MoE layers at full width: through all 61 randomly initialised layers the top-8
    routing of near-uniform router scores flips on rounding noise and the two paths decorrelate (0.8 relative
    difference measured), which says nothing about the kernels."""
    import copy

    import torch

    from batchgen_b200.models.transformer import AttnMeta, Transformer
    from batchgen_b200.models.weights import Linear, ParallelLayout
    from batchgen_b200.parallel.comm import NcclComm
    B = d_ids.shape[0]
    Bl = B // world
    meta = AttnMeta(mode="decode", positions=d_pos, slot_mapping=d_slot, block_table=d_bt, seqlens=d_len)
    rp = model.attn_request_parallel
    model.attn_request_parallel = False
    n_layers = min(len(model.w.layers), n_layers or (model.cfg.first_k_dense + 2))
    all_layers = model.w.layers
    model.w.layers = all_layers[:n_layers]
    try:
        got = model.forward_sp(d_ids, meta, kv).float()
    finally:
        model.w.layers = all_layers
    w = copy.copy(model.w)
    w.layers = []
    for lw in all_layers[:n_layers]:
        lw2 = copy.copy(lw)
        if lw.experts is not None and lw.w13 is not None:       # shared expert of a MoE layer: replicated -> sharded
            I = lw.w2.w.shape[1]
            per = I // world
            if not lw.w13.interleaved or per % 128:
                model.attn_request_parallel = rp
                return {"skipped": "shared-expert weights cannot be cut on quantisation-block boundaries"}
            # rows: the tile-interleaved layout keeps the gate and up rows of 32 output columns together, so a column
            # range is a row range; scales stay in gate-block-rows-then-up-block-rows order
            g0, g1 = rank * per // 128, (rank + 1) * per // 128
            s13 = torch.cat([lw.w13.s[g0:g1], lw.w13.s[I // 128 + g0: I // 128 + g1]], 0).contiguous()
            lw2.w13 = Linear(lw.w13.w[rank * 2 * per:(rank + 1) * 2 * per], s13, interleaved=True)
            lw2.w2 = Linear(lw.w2.w[:, rank * per:(rank + 1) * per].contiguous(), lw.w2.s[:, g0:g1].contiguous())
        w.layers.append(lw2)
    V = model.w.lm_head.shape[0]
    w.lm_head = model.w.lm_head[rank * (V // world):(rank + 1) * (V // world)]
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world)
    base = Transformer(model.cfg, w, layout, NcclComm(), model.rope.max_pos)
    want = base.forward(d_ids, meta, kv).float()[rank * Bl:(rank + 1) * Bl]
    model.attn_request_parallel = rp
    rel = float((got - want).norm() / want.norm())
    agree = float((got.argmax(-1) == want.argmax(-1)).float().mean())
    t = torch.tensor([rel, -agree], device=got.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"max_rel_diff_fused_vs_nccl": float(t[0]), "min_argmax_agreement": float(-t[1]), "rows": B,
            "layers_compared": n_layers}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="deepseek-v3-671b")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--experts", type=int, default=0,
                    help="debug only: fewer routed experts, e.g. 64 on 2 GPUs gives each rank the 32 experts it holds on "
                         "8 (result marked invalid)")
    ap.add_argument("--batch", type=int, default=384, help="decode rows of the whole job")
    ap.add_argument("--prefill-tokens", type=int, default=8192)
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"])
    ap.add_argument("--attn-core", default="auto", choices=["auto", "heads", "requests"],
                    help="decode attention core inside the TP group: split by heads (latent KV replicated) or by "
                         "request (all-to-all of queries/outputs, KV of a row on one rank); auto = requests for N > 1")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="run the decode step eagerly instead of as a CUDA graph")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    ap.add_argument("--profile-ops", default="", help="write a per-operator CUDA-event breakdown to this file")
    ap.add_argument("--bct", action="store_true", help="also run the 512-request workload through the batch API")
    ap.add_argument("--bct-requests", type=int, default=512)
    ap.add_argument("--bct-tokens", type=int, default=1024)
    ap.add_argument("--workload", default="decode", choices=["decode", "distinct64k", "grouped64k", "streamed"],
                    help="decode: the headline decode-step benchmark; the others: long-context DSA workloads "
                         "(use with --model glm-5.3-fp8)")
    ap.add_argument("--requests", type=int, default=2, help="requests of a long-context workload")
    ap.add_argument("--ctx-tokens", type=int, default=65536, help="prompt tokens of a long-context request")
    ap.add_argument("--trace-kernels", default="",
                    help="write the in-step kernel timeline of one captured decode step (start stamps of this "
                         "repository's kernels: period = duration + gap to the next kernel) to this file")
    ap.add_argument("--check-comm", action="store_true",
                    help="N > 1: run one decode step through the NCCL baseline on the same inputs and report the "
                         "largest relative difference of the logits (outside the timed regions)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "streamed":
        return run_streamed(args)
    if args.workload != "decode":
        return run_longctx(args)

    import torch
    import torch.distributed as dist

    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.transformer import AttnMeta
    from batchgen_b200.models.weights import ParallelLayout
    from batchgen_b200.ops import _ext
    from batchgen_b200.ops import sampling as sampling_ops
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.sequence import SamplingParams
    from batchgen_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from batchgen_b200.parallel import make_comm
        comm = make_comm(args.comm, dev)
    _ext.lib()

    cfg = get_model_config(args.model)
    if args.layers:
        cfg.num_layers = args.layers
    if args.experts:
        cfg.n_routed_experts = args.experts
        cfg.n_group = min(cfg.n_group, max(1, args.experts // 8))
        cfg.topk_group = min(cfg.topk_group, cfg.n_group)
    page = 64
    rng = random.Random(1234)
    B = args.batch
    prompt_lens = [rng.randint(512, 4096) for _ in range(B)]
    decoded_so_far = 512                                   # timed at the middle of the 1,024-token decode
    ctx = [p + decoded_so_far for p in prompt_lens]
    e2e_buffer_pages = 4                                   # growth room of each row for the engine-driven steps
    pages_per_seq = [(c + 1 + page - 1) // page for c in ctx]
    total_pages = sum(pages_per_seq) + B * e2e_buffer_pages + 8

    # ---- memory plan: how many distinct expert-weight sets fit next to the KV pool
    fused = comm is not None and getattr(comm, "fused", False)
    layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world, sequence_parallel=fused)
    if fused:
        comm.configure(cfg.hidden_size, cfg.expert_hidden, cfg.n_routed_experts, cfg.num_experts_per_tok,
                       max_tokens=max(B, args.prefill_tokens),
                       a2a_bytes=B * (cfg.num_heads // world) * cfg.kv_cache_dim * 2 if cfg.is_mla else 0)
    n_moe = cfg.num_layers - cfg.first_k_dense
    expert_bytes_layer = (cfg.n_routed_experts // world) * 3 * cfg.moe_intermediate_size * cfg.hidden_size
    kv_bytes = total_pages * page * cfg.kv_cache_dim * 2 * cfg.num_layers
    prefill_kv_bytes = (args.prefill_tokens + 4 * page) * cfg.kv_cache_dim * 2 * cfg.num_layers
    free_b, total_b = torch.cuda.mem_get_info(dev)
    other = 26e9 / world + 12e9                              # attention/dense/shared/embeddings + workspace
    budget = free_b * 0.94 - kv_bytes - prefill_kv_bytes - other
    sets = int(max(1, min(n_moe, budget // expert_bytes_layer)))
    alias = 0 if sets >= n_moe else sets

    t0 = time.time()
    model = build_model(cfg, device=dev, dtype="bf16", seed=0, layout=layout, comm=comm,
                        max_positions=8192, alias_experts_every=alias, gen_device=dev)
    req_core = world > 1 and args.attn_core in ("auto", "requests") and B % world == 0 and not cfg.has_dsa
    model.attn_request_parallel = req_core
    torch.cuda.synchronize()
    build_s = time.time() - t0

    # ---- the engine owns the page pool; the benchmark's sequences are registered with it (their KV is synthetic)
    ecfg = EngineConfig(page_size=page, max_decode_batch=B, max_prefill_tokens=args.prefill_tokens,
                        enable_cuda_graph=not args.no_graph, cuda_graph_max_bucket_size=B, cuda_graph_num_buckets=1,
                        initial_gpu_page_buffer=e2e_buffer_pages, extension_gpu_page_buffer=2, decision_frequency_pages=2,
                        world_size=world, attn_tp_size=world, ep_size=world, device=str(dev), dtype="bf16",
                        decode_attn_split="requests" if req_core else "heads",
                        moe_comm="fused" if fused else "nccl")
    eng = Engine(model, ecfg, num_gpu_pages=total_pages + (args.prefill_tokens // page + 8))
    kv = eng.kv
    for l in range(kv.kv.shape[0]):                        # one slab per layer that keeps paged KV
        kv.kv[l].normal_(0.0, 0.5)
    gen = torch.Generator().manual_seed(7)
    forced = SamplingParams(max_new_tokens=1024, ignore_eos=True)
    seqs = []
    for i in range(B):
        toks = torch.randint(2, cfg.vocab_size, (ctx[i] + 1,), generator=gen).tolist()
        seqs.append(eng.adopt_sequence(toks[: prompt_lens[i]], toks[prompt_lens[i]:], forced))
    # ---- decode step inputs (device resident for the kernel-timed number)
    ids_h = torch.tensor([s.all_ids[-1] for s in seqs], dtype=torch.int32)
    bt_cols = max(pages_per_seq) + e2e_buffer_pages + 1
    if args.bct:                                           # the batch workload's longest row: 4,096 + forced tokens
        bt_cols = max(bt_cols, (4096 + args.bct_tokens) // page + e2e_buffer_pages + 8)
    bt_h = torch.zeros(B, bt_cols, dtype=torch.int32)
    for i, s in enumerate(seqs):
        bt_h[i, : len(s.gpu_pages)] = torch.tensor(s.gpu_pages, dtype=torch.int32)
    pos_h = torch.tensor(ctx, dtype=torch.int32)
    slot_h = torch.tensor([int(bt_h[i, c // page]) * page + c % page for i, c in enumerate(ctx)], dtype=torch.int64)
    len_h = pos_h + 1
    pin = lambda t: t.pin_memory()
    ids_p, bt_p, pos_p, slot_p, len_p = map(pin, (ids_h, bt_h, pos_h, slot_h, len_h))
    d_ids, d_bt, d_pos, d_slot, d_len = (t.to(dev) for t in (ids_h, bt_h, pos_h, slot_h, len_h))
    out_tok = torch.empty(B, dtype=torch.int32, device=dev)
    tok_pinned = torch.empty(B, dtype=torch.int32).pin_memory()

    Bl = B // world if fused else B
    tok_loc = torch.empty(Bl, dtype=torch.int32, device=dev)

    def run_model(ids, meta):
        """-> greedy tokens of the whole step in out_tok (fused path: own rows sampled, then gathered)."""
        if fused:
            sampling_ops.greedy(model.forward_sp(ids, meta, kv), tok_loc)
            dist.all_gather_into_tensor(out_tok, tok_loc)
        else:
            sampling_ops.greedy(model.forward(ids, meta, kv), out_tok)

    # ---- the decode step as one CUDA graph (whole model forward); sampling and token exchange follow it
    runner = None
    graph_kernels = 0
    if not args.no_graph:
        from batchgen_b200.runtime.graphs import DecodeGraphRunner
        runner = DecodeGraphRunner(model, kv, max_batch=B, max_pages_per_seq=bt_h.shape[1], num_buckets=1,
                                   max_bucket=B, sequence_parallel=fused)
        eng.graph_runner = runner
        pl = [list(s.gpu_pages) for s in seqs]
        runner.stage(ids_h.tolist(), pos_h.tolist(), slot_h.tolist(), len_h.tolist(), pl)
        k0 = _ext.LAUNCHES["count"]
        runner.capture(B)
        graph_kernels = (_ext.LAUNCHES["count"] - k0) // 3      # two warm-up runs + the captured one

    def sample_logits(logits):
        if fused:
            sampling_ops.greedy(logits, tok_loc)
            dist.all_gather_into_tensor(out_tok, tok_loc)
        else:
            sampling_ops.greedy(logits, out_tok)

    def decode_step_graph():
        sample_logits(runner.replay(B, B))
        _ext.LAUNCHES["count"] += graph_kernels

    def decode_step_eager():
        meta = AttnMeta(mode="decode", positions=d_pos, slot_mapping=d_slot, block_table=d_bt, seqlens=d_len)
        run_model(d_ids, meta)

    def decode_step_device():
        if runner is not None:
            decode_step_graph()
        else:
            decode_step_eager()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        decode_step_device()
    _ext.check_status()
    if cfg.is_mla:
        # longest sequences first in the attention work lists (static device buffers: graphs see the new order)
        from batchgen_b200.ops import mla_kernel
        own = ctx[rank * (B // world):(rank + 1) * (B // world)] if req_core else ctx
        mla_kernel.reorder_decode_work(dev, [int(c) for c in own])
        decode_step_device()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    l0 = _ext.LAUNCHES["count"]
    if args.profiler_range:
        torch.cuda.profiler.start()
    ms = timed(decode_step_device, args.steps)
    if args.profiler_range:
        torch.cuda.profiler.stop()
    launches = _ext.LAUNCHES["count"] - l0
    clocks = sampler.stop() if sampler else {}
    _ext.check_status()
    ms_step = ms / args.steps
    decode_tps = B * 1000.0 / ms_step

    if args.profile_ops:                                   # every rank runs the same steps (collectives inside)
        from batchgen_b200.utils.timing import TimingStats
        model.timer = TimingStats()
        for _ in range(2):
            decode_step_eager()
            model.timer.step_done()
        torch.cuda.synchronize()
        dsum = model.timer.summary()
        model.timer = TimingStats()
        if rank == 0:
            with open(args.profile_ops, "w") as f:
                f.write("== decode step: ms per step by operator (CUDA events, eager) ==\n")
                for op, d in dsum.items():
                    f.write(f"{op:32s} {d['ms_per_step']:10.3f} ms  {d['share'] * 100:5.1f}%  calls {d['calls']}\n")
    else:
        dsum = None

    comm_check = None
    if args.check_comm and fused:
        # one eager decode step over the fused kernels against the same step over the NCCL baseline: the fused
        # model's weights are reused (attention shards are the same; the shared experts and lm_head, replicated in
        # the sequence-parallel layout, are sliced to their tensor-parallel shard for the baseline run)
        # dense layers only (no routing: pure rounding noise of the two data paths), then with one and two MoE layers
        comm_check = {f"layers_{n}": compare_with_nccl(model, kv, d_ids, d_pos, d_slot, d_bt, d_len, rank, world, dist, n)
                      for n in (cfg.first_k_dense, cfg.first_k_dense + 1, cfg.first_k_dense + 2)}

    e2e = None
    if not args.no_e2e:
        # K real decode steps through the engine: admission, input staging from pinned memory, graph replay,
        # sampling, token exchange, token read-back on the host every step
        done = eng.decode_steps(max(args.warmup, 3))
        assert done == max(args.warmup, 3), f"engine warm-up ran {done} steps"
        _ext.check_status()
        l1 = _ext.LAUNCHES["count"]
        steps_run = []
        ms_e = timed(lambda: steps_run.append(eng.decode_steps(args.steps)), 1) / args.steps
        assert steps_run == [args.steps], f"engine ran {steps_run} steps, wanted {args.steps}"
        _ext.check_status()
        h2d = runner.h2d_bytes_per_step if runner is not None else B * (4 + 4 + 8 + 4) + bt_h.numel() * 4
        e2e = {"value": B * 1000.0 / ms_e, "unit": "decode tokens/s", "ms_per_step": ms_e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": B * 4, "api": "Engine.decode_steps",
               "launches_outside_graph": _ext.LAUNCHES["count"] - l1}

    prefill = None
    if not args.no_prefill:
        # one packed prefill micro-batch of sequences of 2,048 tokens through all layers
        n_seq = max(1, args.prefill_tokens // 2048)
        L = args.prefill_tokens // n_seq
        T = n_seq * L
        pp = (L + page - 1) // page
        pbt = torch.tensor(kv.alloc.alloc(n_seq * pp), dtype=torch.int32).view(n_seq, pp).to(dev)
        ppos = torch.arange(L, dtype=torch.int32).repeat(n_seq).to(dev)
        pslot = torch.cat([(pbt[i].long().repeat_interleave(page)[:L] * page
                            + torch.arange(L, device=dev) % page) for i in range(n_seq)])
        pids = torch.randint(2, cfg.vocab_size, (T,), generator=gen, dtype=torch.int32).to(dev)
        cu = [i * L for i in range(n_seq + 1)]
        rows = torch.tensor([c - 1 for c in cu[1:]], device=dev)

        def prefill_step():
            meta = AttnMeta(mode="prefill", positions=ppos, slot_mapping=pslot, block_table=pbt, cu_seqlens=cu,
                            ctx_lens=[0] * n_seq, logit_rows=rows)
            if fused:
                sampling_ops.greedy(model.forward_sp(pids, meta, kv))
            else:
                sampling_ops.greedy(model.forward(pids, meta, kv))

        prefill_step()
        torch.cuda.synchronize()
        _ext.check_status()
        psum = None
        if args.profile_ops:
            model.timer.reset()
            prefill_step()
            model.timer.step_done()
            torch.cuda.synchronize()
            psum = model.timer.summary()
            from batchgen_b200.utils.timing import null_timer
            model.timer = null_timer()
        if args.profile_ops and rank == 0:
            with open(args.profile_ops, "a") as f:
                f.write("== prefill micro-batch: ms per step by operator (CUDA events, eager) ==\n")
                for op, d in psum.items():
                    f.write(f"{op:32s} {d['ms_per_step']:10.3f} ms  {d['share'] * 100:5.1f}%  calls {d['calls']}\n")
        ms_p = timed(prefill_step, 2) / 2
        _ext.check_status()
        prefill = {"tokens_per_s": T * 1000.0 / ms_p, "ms_per_microbatch": ms_p, "tokens": T, "seq_len": L}
        kv.alloc.free(pbt.flatten().tolist())

    if args.trace_kernels:
        from batchgen_b200.utils import kernel_trace
        tbuf = kernel_trace.enable(dev)
        barrier()
        decode_step_device()
        barrier()
        kernel_trace.disable(dev)
        if rank == 0:
            recs = kernel_trace.read(tbuf)
            rows = kernel_trace.summarize(recs)
            with open(args.trace_kernels, "w") as f:
                span = (recs[-1][0] - recs[0][0]) / 1e3 if recs else 0.0
                f.write(f"== one captured decode step: {len(recs)} stamped kernels over {span:.1f} us ==\n")
                for r in rows:
                    f.write(f"{r['kernel']:36s} {r['launches']:6d} launches {r['us']:10.1f} us {r['share'] * 100:5.1f}%"
                            f"  {r['us'] / max(r['launches'], 1):8.2f} us each\n")
                f.write("== first layers in order (us since the first stamp, kernel) ==\n")
                for t, tag, line in recs[:140]:
                    f.write(f"{(t - recs[0][0]) / 1e3:10.2f}  {kernel_trace.kernel_name(tag, line)}\n")
    bct = None
    if args.bct:
        if rank == 0:                                   # the step numbers survive a failure of the long workload
            print(json.dumps({"partial": True, "ms_per_step": ms_step, "value": decode_tps, "e2e": e2e,
                              "prefill": prefill, "comm_check": comm_check}), file=sys.stderr, flush=True)
        try:
            bct = run_bct(eng, cfg, args, rank, world, barrier)
        except Exception as exc:                        # noqa: BLE001 - reported in the result line
            bct = {"error": f"{type(exc).__name__}: {exc}"[:400]}

    if rank == 0:
        total_prompt = sum(rng.randint(512, 4096) for _ in range(512))
        bct_proj = None
        if prefill:
            bct_proj = total_prompt / prefill["tokens_per_s"] + 512 * 1024 / decode_tps
        out = {
            "metric": "decode tokens/s (DeepSeek-V3-671B FP8, batch workload of BASELINE config 2)",
            "value": decode_tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8(e4m3 block-scaled weights+activations)/bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "global_batch": B,
                       "seq_len": int(sum(ctx) / len(ctx)), "prompt_lens": "U[512,4096]", "decoded_so_far": 512,
                       "parallelism": f"tp{world}+ep{world}",
                       "attn_core": ("head-sharded projections (TP), decode core split by request with an all-to-all "
                                     "inside the TP group" if req_core else "split by heads"),
                       "comm": ("fused-nvlink-kernels" if fused else "nccl") if world > 1 else "none",
                       "distinct_expert_sets": sets, "moe_layers": n_moe, "cuda_graph": runner is not None,
                       "l2_note": "inputs (weights + KV, tens of GB per step) exceed the 126 MB L2",
                       "valid": not (args.layers or args.experts), "build_seconds": round(build_s, 1)},
            "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "prefill": prefill,
            "bct_projected_s": bct_proj, "bct": bct, "comm_check": comm_check,
        }
        print(json.dumps(out))
    sys.stdout.flush()
    if world > 1:
        # graphs that captured collectives go first; a stuck teardown must not outlive the result
        import gc
        import threading
        threading.Timer(20.0, lambda: os._exit(0)).start()
        runner = None
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
