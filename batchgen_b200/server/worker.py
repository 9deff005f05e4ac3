"""Worker process: one per GPU (or one CPU process), running the engine's scheduling loop and talking to
the server over two ``multiprocessing`` queues.

Messages down (server -> rank 0):  ``{"type": "admit", "entries": [{slot, batch_id, request_id, prompt_ids,
sampling}]}``, ``{"type": "cancel", "batch_id"}``, ``{"type": "shutdown"}``.
Messages up (rank 0 -> server): ``{"type": "ready" | "deployment_capacity" | "completion" | "worker_fatal" |
"heartbeat", ...}``.

All ranks run in lock step: rank 0 drains its queue once per loop iteration and broadcasts the message list
(``broadcast_object_list``; a one-element list when idle doubles as the heartbeat), every rank applies the
same admissions and takes the same engine step.  Ordered teardown: the engine stops at a step boundary, the
process group is destroyed, queues are flushed.

Reference parity: batchgen/server_worker_main_loop.py:574-1083 (entry, NCCL env, rendezvous, warm-up,
readiness, main loop with rank-0 poll + broadcast, fatal sideband, teardown), batchgen/server/process_utils.py:38
(``die_with_parent``).
"""
from __future__ import annotations

import ctypes
import os
import queue as queue_mod
import signal
import sys
import time
import traceback
from typing import Any, Dict, List, Optional


def die_with_parent() -> None:
    """Ask the kernel to SIGKILL this process when its parent dies (Linux PR_SET_PDEATHSIG)."""
    try:
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        libc.prctl(1, signal.SIGKILL, 0, 0, 0)
    except OSError:
        pass


def setup_nccl_env() -> None:
    """NCCL settings for a single NVSwitch node.  NVLS stays at NCCL's default here (the reference turns it
    off because registering buffers with the switch made graph capture slow, server_worker_main_loop.py:553-571)."""
    os.environ.setdefault("TORCH_NCCL_ENABLE_MONITORING", "0")
    os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo")
    if os.environ.get("BATCHGEN_DETERMINISTIC") == "1":
        os.environ.setdefault("NCCL_ALGO", "allreduce:tree")


_STORES: list = []


def _memory_profile(device: str) -> Dict[str, Any]:
    """Device and host memory of this worker for the heartbeat: allocator counters on a GPU, resident set size."""
    out: Dict[str, Any] = {}
    try:
        import resource
        out["host_rss_mb"] = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss // 1024
    except (ImportError, OSError):
        pass
    if device.startswith("cuda"):
        import torch
        free, total = torch.cuda.mem_get_info(torch.device(device))
        out.update(device_allocated_mb=torch.cuda.memory_allocated(device) >> 20,
                   device_reserved_mb=torch.cuda.memory_reserved(device) >> 20,
                   device_peak_mb=torch.cuda.max_memory_allocated(device) >> 20,
                   device_free_mb=free >> 20, device_total_mb=total >> 20)
    return out


def build_engine(args, rank: int, world: int, device: str, phases=None, phase_slot: Optional[int] = None):
    import torch

    from ..config import get_model_config
    from ..models import build_model
    from ..models.weights import ParallelLayout
    from ..runtime.engine import Engine
    from ..runtime.planner import size_kv_pool

    cfg = get_model_config(args.model)
    ecfg = args.engine_config()
    ecfg.device = device
    dtype = "bf16" if device.startswith("cuda") else "fp32"
    loader = None
    if getattr(args, "param_store_path", "") and getattr(args, "param_store_index", None):
        # the server read the checkpoint once into a node-shared region: attach and serve tensors as views
        from ..core import native
        store = native.ParameterStore(fd=os.open(args.param_store_path, os.O_RDONLY), read_only=True)
        store.import_index(args.param_store_index)
        loader = store.loader()
        _STORES.append(store)                         # the mapping must outlive the tensors built from it
    elif args.converted_ckpt_dir:
        from ..ckpt.converter import ConvertedCheckpoint
        loader = ConvertedCheckpoint(args.converted_ckpt_dir).loader()
    comm = None
    layout = ParallelLayout()
    fused = False
    if world > 1:
        from ..models.transformer import Transformer
        from ..parallel import make_comm
        why_not = Transformer.supports_sequence_parallel(cfg) if device.startswith("cuda") else "no GPU"
        fused = args.moe_comm == "fused" and why_not is None
        if args.moe_comm == "fused" and not fused:
            from ..utils import eventlog
            eventlog.get_log().info("worker.comm", rank=rank, chosen="nccl", reason=why_not)
        comm = make_comm("fused" if fused else "nccl", device if fused else None)
        layout = ParallelLayout(tp_rank=rank, tp_size=world, ep_rank=rank, ep_size=world, sequence_parallel=fused)
    if getattr(args, "decode_attn_split", "heads") == "auto" and fused and cfg.is_mla and not cfg.has_dsa:
        # the latent KV of a row is shared by all heads: on the fused path each rank attends over its own rows with
        # every head (two chunked exchanges per layer) instead of streaming every row's KV for its own heads
        ecfg.decode_attn_split = "requests"
    model = build_model(cfg, device=device, dtype=dtype, seed=args.seed, layout=layout, comm=comm, loader=loader,
                        max_positions=max(8192, args.max_model_len if args.max_model_len > 0 else 8192))
    if world > 1 and ecfg.decode_attn_split == "requests" and cfg.is_mla and not cfg.has_dsa:
        model.attn_request_parallel = True       # the engine pins every sequence to an owner rank (Engine._owner_layout)
    if fused:
        # steps of the fused path are bounded by the symmetric heap: cap the packed prefill micro-batch
        ecfg.max_prefill_tokens = min(ecfg.max_prefill_tokens, args.fused_max_tokens)
        step_rows = max(ecfg.max_prefill_tokens, ecfg.max_decode_batch + 8 * world)
        a2a = 0
        if model.attn_request_parallel:
            a2a = (ecfg.max_decode_batch + 8 * world) * (cfg.num_heads // world) * cfg.kv_cache_dim * 2
        comm.configure(cfg.hidden_size, cfg.expert_hidden, cfg.n_routed_experts, cfg.num_experts_per_tok,
                       max_tokens=step_rows, a2a_bytes=a2a)
    phase_slot = rank if phase_slot is None else phase_slot
    if phases is not None:
        phases.enter(phase_slot, "kv-pool")
    pages, host_pages = size_kv_pool(cfg, ecfg, device, model.dtype)
    host_fd = None
    if getattr(args, "host_kv_region", "") and device.startswith("cuda"):
        host_fd = os.open(args.host_kv_region, os.O_RDWR)      # the server's region: same pages for every worker
    eng = Engine(model, ecfg, num_gpu_pages=pages, num_host_pages=host_pages, host_kv_fd=host_fd)
    if device.startswith("cuda") and ecfg.enable_cuda_graph:
        if phases is not None:
            phases.enter(phase_slot, "graph-capture")
        from ..runtime.graphs import DecodeGraphRunner
        max_pages = -(-eng.kv_token_budget // ecfg.page_size)
        eng.graph_runner = DecodeGraphRunner(model, eng.kv, max_batch=ecfg.max_decode_batch,
                                             max_pages_per_seq=min(max_pages, pages),
                                             num_buckets=ecfg.cuda_graph_num_buckets,
                                             max_bucket=ecfg.cuda_graph_max_bucket_size, sequence_parallel=fused)
    return cfg, eng


def worker_main(rank: int, world: int, args, request_queue, response_queue, ready_event, shutdown_flag,
                feed_counter=None) -> None:
    """Entry point of a worker process (also callable in-process for tests)."""
    die_with_parent()
    from . import run_guard
    run_lock = run_guard.join_run(args)               # noqa: F841 - held (shared) until the process exits
    from ..utils import eventlog
    log = eventlog.configure_process(f"worker{rank}", args.log_dir or None, args.log_level,
                                     flight_recorder=bool(args.log_dir))
    import torch
    import torch.distributed as dist

    dp_rank = int(getattr(args, "dp_rank", 0))
    gpu = int(getattr(args, "gpu_offset", 0)) + rank          # data-parallel cohorts own consecutive GPUs
    slot = int(getattr(args, "startup_slot_base", 0)) + rank

    def up(msg: Dict[str, Any]) -> None:
        if rank == 0:
            msg["cohort"] = dp_rank
            response_queue.put(msg)

    from .startup_phases import record_of
    phases = record_of(args)
    import faulthandler
    try:                                                  # SIGUSR1 -> stack dump of every thread (watchdog asks for it)
        stack_file = open(os.path.join(args.log_dir, f"worker{rank}.stacks"), "a") if args.log_dir else sys.stderr
        faulthandler.register(signal.SIGUSR1, file=stack_file, all_threads=True)
    except (OSError, ValueError, AttributeError):
        pass
    try:
        use_cuda = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
        device = f"cuda:{gpu}" if use_cuda else "cpu"
        if use_cuda:
            torch.cuda.set_device(gpu)
        phases.enter(slot, "communicator-init")
        if world > 1:
            setup_nccl_env()
            dist.init_process_group("nccl" if use_cuda else "gloo", init_method=f"tcp://{args.dist_init_addr}",
                                    rank=rank, world_size=world)
            t = torch.ones(1, device=device)
            dist.all_reduce(t)                        # warm-up: the first collective builds the communicators
        from ..runtime.sequence import SamplingParams
        phases.enter(slot, "model-build")
        cfg, eng = build_engine(args, rank, world, device, phases=phases, phase_slot=slot)
        phases.enter(slot, "prewarm")
        log.info("worker.ready", rank=rank, device=device, gpu_pages=eng.kv.num_pages,
                 host_pages=eng.host_kv.num_pages if eng.host_kv else 0)
        up({"type": "deployment_capacity", "gpu_pages": eng.kv.num_pages, "page_size": eng.buf.page_size,
            "kv_token_budget": eng.kv_token_budget, "max_decode_batch": eng.ecfg.max_decode_batch,
            "model": cfg.name, "vocab_size": cfg.vocab_size})
        if world > 1:
            dist.barrier()
        phases.enter(slot, "serving")
        if rank == 0:
            ready_event.set()

        by_idx: Dict[int, Dict[str, Any]] = {}
        cancelled = set()
        adopt: List[Dict[str, Any]] = []              # rows handed over by another cohort, waiting for host pages
        # BATCHGEN_PROFILE_STEPS=first:last brackets those engine steps with the profiler API for an attached profiler;
        # BATCHGEN_MEMORY_HISTORY=<dir> records allocator events and writes a snapshot when a step runs out of memory
        from ..utils.capture_window import CaptureWindow, MemoryHistory
        window, mem_history = CaptureWindow.from_env(), MemoryHistory.from_env()
        # the token book: prompts live once per node in a shared int32 table; rank 0 binds a slot and writes the
        # prompt, the step broadcast then carries (offset, length) instead of the tokens, and completions are read
        # back from the book (batchgen/query_book.py, batchgen/batchgen_worker.py: node-shared token memfd)
        from ..runtime.query_book import NodeSharedTokens, QueryBook
        qb_tokens = max(int(getattr(args, "query_book_mb", 64)), 1) * (1 << 20) // 4
        qb_rows = max(qb_tokens // 4096, 4)
        handle = [None]
        shared = None
        if rank == 0:
            shared = NodeSharedTokens.create(qb_rows, 4096)
            handle[0] = shared.handle()
        if world > 1:
            dist.broadcast_object_list(handle, src=0)
            if rank != 0:
                shared = NodeSharedTokens.attach(tuple(handle[0]))
        book = QueryBook(qb_rows * 4096 * 4, page_tokens=4096, storage=shared.tensor)   # rank 0 allocates and writes
        flat = shared.tensor.view(-1)

        def on_complete(seq) -> None:
            meta = by_idx.pop(seq.global_idx, None)
            if meta is None:
                return
            reason = "cancelled" if meta["batch_id"] in cancelled else seq.finish_reason
            out_ids = list(seq.output_ids)
            if rank == 0 and meta.get("qb_slot") is not None:
                qs = meta["qb_slot"]
                room = book.metadata(qs).remaining
                book.append_tokens([qs] * min(len(out_ids), room), out_ids[:room])
                if room >= len(out_ids):
                    out_ids = book.generated_tokens(qs).tolist()       # the book is the record of the trajectory
                book.release(qs)
            up({"type": "completion", "slot": meta["slot"], "batch_id": meta["batch_id"],
                "request_id": meta["request_id"], "output_ids": out_ids,
                "prompt_tokens": len(seq.prompt_ids), "cached_tokens": seq.cached_prefix_tokens,
                "finish_reason": reason})

        eng.on_complete = on_complete
        if feed_counter is not None:
            eng.step_hook = lambda phase: feed_counter.__setattr__("value", feed_counter.value + 1)
        stuck = float(args.watchdog_test_stuck_time or 0.0)
        last_beat = time.monotonic()
        running = True
        while running:
            msgs: List[Dict[str, Any]] = []
            if rank == 0:
                try:
                    block = not eng.has_work()
                    m = request_queue.get(timeout=0.2) if block else request_queue.get_nowait()
                    msgs.append(m)
                    while len(msgs) < 64:
                        msgs.append(request_queue.get_nowait())
                except queue_mod.Empty:
                    pass
                if shutdown_flag.is_set():
                    msgs.append({"type": "shutdown"})
                for m in msgs:                          # prompts move into the book; the broadcast carries references
                    if m.get("type") != "admit":
                        continue
                    for e in m["entries"]:
                        ids = e.get("prompt_ids")
                        want = len(ids or ()) + int(e["sampling"].get("max_new_tokens", 0)) + 1
                        uid = f'{e["batch_id"]}/{e["request_id"]}/{e["slot"]}'
                        if not ids or book.has_sequence(uid) or not book.can_reserve(want):
                            continue                     # no room (or a bad request): the tokens travel inline
                        qs = book.bind(uid, want)
                        book.write_prompt(qs, torch.tensor(ids, dtype=torch.int32))
                        e["qb"] = (qs, book._base(qs), len(ids))
                        e["prompt_ids"] = None
            if world > 1:
                box = [msgs]
                dist.broadcast_object_list(box, src=0)
                msgs = box[0]
            for m in msgs:
                kind = m.get("type")
                if kind == "shutdown":
                    running = False
                elif kind == "end_session":
                    eng.end_session(m["session_id"])
                elif kind == "migrate_out":
                    # hand parked rows to another cohort: every rank of this cohort packs its copy of the same rows
                    # (the scheduler is the same on all of them) into one file per row and rank
                    from ..runtime import kv_migration
                    moved = []
                    rows = [r for r in kv_migration.parked_rows(eng) if not r.session_id and r.global_idx in by_idx]
                    for i, s_row in enumerate(rows[: int(m.get("count", 1))]):
                        if not kv_migration.can_export(eng):
                            break
                        meta = by_idx.pop(s_row.global_idx)
                        stem = os.path.join(m["dir"], f'{m["ticket"]}_{i}')
                        n_pages = len(s_row.host_pages)
                        torch.save(kv_migration.export_sequence(eng, s_row), f"{stem}.r{rank}.pt")
                        if rank == 0 and meta.get("qb_slot") is not None:
                            book.release(meta["qb_slot"])            # the payload carries the tokens from here on
                        moved.append({"stem": stem, "pages": n_pages,
                                      "meta": {"slot": meta["slot"], "batch_id": meta["batch_id"],
                                               "request_id": meta["request_id"]}})
                    up({"type": "migrated_out", "ticket": m["ticket"], "rows": moved, "dst": m.get("dst")})
                elif kind == "migrate_in":
                    from ..runtime import kv_migration
                    adopt.extend(m["rows"])
                elif kind == "cancel":
                    cancelled.add(m["batch_id"])
                    for s in list(eng.seqs.values()):
                        if s.batch_id == m["batch_id"] and s.status.name != "COMPLETED":
                            s.params.max_new_tokens = max(1, s.num_decoded)   # finishes at the next boundary
                elif kind == "admit":
                    for e in m["entries"]:
                        try:
                            sp = SamplingParams(**e["sampling"])
                            ids, qs = e["prompt_ids"], None
                            if e.get("qb") is not None:
                                qs, base, n = e["qb"]
                                ids = flat[base:base + n].tolist()
                            s = eng.add_request(ids, sp, custom_id=e["request_id"], batch_id=e["batch_id"],
                                                session_id=e.get("session_id"))
                            by_idx[s.global_idx] = {"slot": e["slot"], "batch_id": e["batch_id"],
                                                    "request_id": e["request_id"], "qb_slot": qs}
                        except Exception as ex:  # noqa: BLE001  (bad request: report, keep serving)
                            if rank == 0 and e.get("qb") is not None:
                                book.release(e["qb"][0])
                            up({"type": "completion", "slot": e["slot"], "batch_id": e["batch_id"],
                                "request_id": e["request_id"], "output_ids": [], "prompt_tokens": 0,
                                "cached_tokens": 0, "finish_reason": f"error: {ex}"})
            for row in list(adopt):
                # adopt rows another cohort handed over; a full host tier makes the row wait for the next round
                from ..runtime import kv_migration
                from ..runtime.kv_cache import OutOfPages
                path = f'{row["stem"]}.r{rank}.pt'
                try:
                    s_new = kv_migration.import_sequence(eng, torch.load(path, weights_only=True), rank)
                except OutOfPages:
                    continue
                by_idx[s_new.global_idx] = dict(row["meta"], qb_slot=None)
                adopt.remove(row)
                try:
                    os.remove(path)
                except OSError:
                    pass
                log.info("worker.adopted_row", rank=rank, request=row["meta"]["request_id"], pages=row["pages"])
            if not running:
                break
            if stuck > 0 and eng.has_work():
                time.sleep(stuck)                      # host-side fault injection for the watchdog test
                stuck = 0.0
            if eng.has_work():
                window.before_step()
                try:
                    eng.step()
                except Exception as ex:  # noqa: BLE001 - re-raised: only the allocator snapshot is added here
                    if "out of memory" in str(ex).lower():
                        snap = mem_history.dump("oom")
                        if snap:
                            log.error("worker.memory_snapshot", rank=rank, path=snap)
                    raise
                window.after_step()
                if feed_counter is not None:
                    feed_counter.value += 1
                # completed sequences are dropped so that the table does not grow without bound
                for gi in [g for g, s in eng.seqs.items() if s.status.name == "COMPLETED"]:
                    del eng.seqs[gi]
            if rank == 0 and time.monotonic() - last_beat > float(getattr(args, "heartbeat_interval", 5.0)):
                last_beat = time.monotonic()
                from ..runtime import kv_migration
                up({"type": "heartbeat", "ts": time.time(), "live": len(eng.seqs), "free_pages": eng.kv.alloc.num_free,
                    "parked": len([r for r in kv_migration.parked_rows(eng) if not r.session_id]),
                    "host_free": eng.host_kv.alloc.num_free if eng.host_kv is not None else 0,
                    "stats": eng.stats.summary(), "steps": eng.step_ring.summary(), "memory": _memory_profile(device),
                    "query_book": {"active": book.active_count,
                                                                  "free_pages": book.free_page_count}})
        log.info("worker.shutdown", rank=rank)
    except Exception as ex:  # noqa: BLE001
        log.error("worker.fatal", rank=rank, error=str(ex), trace=traceback.format_exc()[-1500:])
        recent = eng.step_ring.tail(8) if "eng" in locals() else []
        response_queue.put({"type": "worker_fatal", "rank": rank, "cohort": dp_rank, "error": f"{type(ex).__name__}: {ex}",
                            "recent_steps": recent})
        raise
    finally:
        try:
            if world > 1 and dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
        log.close()
