"""BatchScheduler: from an uploaded JSONL file to a published output file.

``enqueue(batch)`` hands a batch to a preparation thread that validates the file, builds prompts (chat
template + tokeniser, in a thread pool), registers a ``BatchTracker`` and submits the requests to the
``IntakePool`` all-or-nothing.  A drain thread moves requests from the intake pool into free
``SchedulingPool`` slots and sends ``admit`` messages to the workers; a completion pump reads worker
messages, detokenises, appends the result line to the batch's incremental output (fsync per line), counts it
once, and finalises the batch when its last request is in: the output is published as a file object and the
batch turns ``completed``.  Requests rejected individually (bad sampling values, prompt beyond the context
budget) become ``error`` items in the same output file.  ``submit_turn`` runs one request synchronously for the
session API.

Reference parity: batchgen/server/batch_scheduler.py (``_process_batch`` :617, prompt building :761-1000, pool
mode :1380-1507, drain loop :1597-1690, completion listener :1762, output writing :2035, finalisation :2184).
"""
from __future__ import annotations

import concurrent.futures
import os
import queue as queue_mod
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from ..runtime import batch_api
from ..runtime.sequence import Sequence
from .io_struct import BatchError, BatchErrors, BatchObject
from .pools import NORMAL, IntakeFull, IntakePool, IntakeRequest, SchedulingPool
from .storage import StorageManager


class BatchScheduler:
    def __init__(self, storage: StorageManager, worker, args, tokenizer):
        self.storage, self.worker, self.args, self.tok = storage, worker, args, tokenizer
        self.intake = IntakePool(args.max_intake_capacity)
        self.pool = SchedulingPool(args.scheduling_slots)
        self._prep_q: "queue_mod.Queue" = queue_mod.Queue()
        self._threads: List[threading.Thread] = []
        self._stop = threading.Event()
        self._quiesced = threading.Event()
        self._reqs: Dict[str, Dict[str, batch_api.BatchRequest]] = {}
        self._opts: Dict[str, batch_api.BatchOptions] = {}
        self._turn_waiters: Dict[str, "queue_mod.Queue"] = {}
        self._lock = threading.RLock()
        self._tok_pool = concurrent.futures.ThreadPoolExecutor(max_workers=4, thread_name_prefix="tokenise")
        self.capacity: Optional[Dict[str, Any]] = None
        dp = max(1, int(getattr(args, "dp_size", 1)))
        self._dp_load = [0] * dp                      # running sum of prompt length^2 of the requests in flight
        self._slot_cost: Dict[int, Any] = {}          # pool slot -> (cohort, cost) until the completion arrives
        self._session_cohort: Dict[str, int] = {}
        self.dp_assigned = [0] * dp                   # requests handed to each cohort so far
        self.last_heartbeat: Optional[Dict[str, Any]] = None
        # hand-over of parked rows between cohorts (runtime.kv_migration.export_sequence / import_sequence)
        self._cohort_stats: Dict[int, Dict[str, int]] = {}
        self._handover: Dict[str, Any] = {}           # ticket -> (source, destination, time asked)
        self.migrated_rows = 0

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        for name, fn in (("batch-prepare", self._prepare_loop), ("intake-drain", self._drain_loop),
                         ("completion-pump", self._completion_loop)):
            t = threading.Thread(target=fn, name=name, daemon=True)
            t.start()
            self._threads.append(t)

    def stop(self) -> None:
        self._stop.set()
        self._prep_q.put(None)
        for t in self._threads:
            t.join(timeout=3)
        self._tok_pool.shutdown(wait=False)

    def quiesce(self) -> None:
        self._quiesced.set()

    def resume(self) -> None:
        self._handover.clear()              # a replaced cohort neither answers an open hand-over nor keeps its counters
        self._cohort_stats.clear()
        self._quiesced.clear()

    def has_work(self) -> bool:
        return self.pool.used > 0

    def rebind_queues(self, request_queue, response_queue) -> None:
        pass        # queues are read through self.worker on every use

    # ------------------------------------------------------------------ intake
    def enqueue(self, batch: BatchObject) -> None:
        self._prep_q.put(batch.id)

    def _tool_call_format(self) -> str:
        """The tool-call markup of the served model's family (``runtime.output_parsers``)."""
        from ..config import get_model_config
        from ..runtime.output_parsers import FAMILY_FORMAT
        try:
            return FAMILY_FORMAT.get(get_model_config(self.args.model).family, "json")
        except KeyError:
            return "json"

    def _fail_batch(self, b: BatchObject, code: str, message: str, line: Optional[int] = None) -> None:
        b.status = "failed"
        b.failed_at = int(time.time())
        b.errors = BatchErrors(data=[BatchError(code=code, message=message, line=line)])
        fo = self.storage.publish_output(b.id)
        if fo is not None:
            b.output_file_id = fo.id
        self.storage.save_batch(b)

    def _prepare_loop(self) -> None:
        while not self._stop.is_set():
            bid = self._prep_q.get()
            if bid is None:
                return
            b = self.storage.get_batch(bid)
            if b is None or b.status != "validating":
                continue
            try:
                self._process_batch(b)
            except Exception as e:  # noqa: BLE001
                self._fail_batch(b, "internal_error", f"{type(e).__name__}: {e}")

    def _process_batch(self, b: BatchObject) -> None:
        data = self.storage.read_file(b.input_file_id)
        if data is None:
            return self._fail_batch(b, "file_not_found", f"input file {b.input_file_id} does not exist")
        try:
            reqs = batch_api.parse_batch_lines(data.decode("utf-8", errors="replace").splitlines(), b.endpoint)
        except batch_api.BatchFormatError as e:
            return self._fail_batch(b, "invalid_file", str(e))
        opts = batch_api.BatchOptions(endpoint=b.endpoint, max_decoding_length=b.max_decoding_length or 256,
                                      temperature=b.temperature, top_p=b.top_p, top_k=b.top_k,
                                      parse_thinking=self.args.parse_thinking, parse_tool_call=self.args.parse_tool_call,
                                      include_special_tokens=self.args.detokenization_include_special_tokens,
                                      model=self.args.model, tool_call_format=self._tool_call_format())
        budget = (self.capacity or {}).get("kv_token_budget")

        def build(req):
            try:
                ids = batch_api.prompt_ids(req, self.tok)
                sp = batch_api.sampling_from_body(req.body, opts)
                if not ids:
                    raise ValueError("empty prompt")
                if budget and len(ids) + sp.max_new_tokens > budget:
                    raise ValueError(f"prompt of {len(ids)} tokens + {sp.max_new_tokens} new tokens exceeds the "
                                     f"context budget {budget}")
                return req, ids, sp, None
            except Exception as e:  # noqa: BLE001
                return req, None, None, str(e)

        built = list(self._tok_pool.map(build, reqs))
        with self._lock:
            self._reqs[b.id] = {r.custom_id: r for r in reqs}
            self._opts[b.id] = opts
        self.pool.register_batch(b.id, len(reqs))
        b.request_counts.total = len(reqs)
        good = [IntakeRequest(b.id, r.custom_id, ids, sp.__dict__.copy(), NORMAL) for r, ids, sp, err in built if err is None]
        try:
            self.intake.submit_batch(good)
        except IntakeFull as e:
            self.pool.trackers.pop(b.id, None)
            return self._fail_batch(b, "intake_full", str(e))
        b.status = "in_progress"
        b.in_progress_at = int(time.time())
        self.storage.save_batch(b)
        for r, ids, sp, err in built:
            if err is not None:
                self._record(b.id, r.custom_id, batch_api.error_item(r, err), ok=False)

    # ------------------------------------------------------------------ drain to workers
    def _drain_loop(self) -> None:
        while not self._stop.wait(0.02):
            if self._quiesced.is_set() or self.worker.state != "ready":
                continue
            picked = self.pool.select_from_intake(self.intake)
            if not picked:
                continue
            dp = getattr(self.worker, "dp", 1)
            cohorts = [0] * len(picked)
            if dp > 1:
                # data parallelism: longest prompts first, each to the cohort with the smallest running sum of
                # length^2 (prefill cost); a session stays with the cohort that holds its context
                # (batchgen/batchgen_worker.py:1987-2033)
                cohorts = self._assign_cohorts([r.prompt_ids for _, r in picked], dp)
                for i, (slot, r) in enumerate(picked):
                    sid = r.meta.get("session_id")
                    if sid:
                        cohorts[i] = self._session_cohort.setdefault(sid, cohorts[i])
                    cost = len(r.prompt_ids) ** 2
                    self._dp_load[cohorts[i]] += cost
                    self._slot_cost[slot] = (cohorts[i], cost)
                    self.dp_assigned[cohorts[i]] += 1
            for c in sorted(set(cohorts)):
                entries = [{"slot": s, "batch_id": r.batch_id, "request_id": r.request_id, "prompt_ids": r.prompt_ids,
                            "sampling": r.sampling, "session_id": r.meta.get("session_id")}
                           for (s, r), cc in zip(picked, cohorts) if cc == c]
                self.worker.send({"type": "admit", "entries": entries}, cohort=c)

    def _assign_cohorts(self, prompts: List[List[int]], dp: int) -> List[int]:
        """Cohort of each request of one drain.  With prefix reuse on, prompts that share their first page travel
        together (a cohort computes the shared prefix once; a family is split only when that lowers the predicted
        makespan: ``wave_plan.pack_wave_ranks``); otherwise every prompt goes, longest first, to the cohort with the
        smallest running sum of squared lengths."""
        if getattr(self.args, "enable_prefix_cache", False) and len(prompts) > 1:
            from ..runtime.wave_plan import pack_wave_ranks
            return list(pack_wave_ranks(prompts, dp, int(getattr(self.args, "page_size", 64)),
                                        initial_load=self._dp_load).rank_of)
        from ..runtime.scheduler import assign_ranks_l2
        return assign_ranks_l2([len(p) for p in prompts], dp, initial_load=self._dp_load)

    # ------------------------------------------------------------------ completions
    def _completion_loop(self) -> None:
        while not self._stop.is_set():
            try:
                m = self.worker.response_queue.get(timeout=0.1)
            except (queue_mod.Empty, OSError, ValueError):
                continue
            kind = m.get("type")
            if kind == "completion":
                self._on_completion(m)
            elif kind == "deployment_capacity":
                self.capacity = m
                self.worker.capacity = m
            elif kind == "heartbeat":
                self.last_heartbeat = m
                self._cohort_stats[int(m.get("cohort", 0))] = {k: int(m.get(k, 0)) for k in ("parked", "live", "host_free")}
                self._maybe_hand_over()
            elif kind == "migrated_out":
                self._on_migrated_out(m)
            elif kind == "worker_fatal":
                self.worker.last_error = m.get("error")

    # ------------------------------------------------------------------ hand-over between cohorts
    def _handover_dir(self) -> str:
        import tempfile
        d = os.path.join(getattr(self.args, "runtime_dir", "") or tempfile.gettempdir(), "handover")
        os.makedirs(d, exist_ok=True)
        return d

    def _maybe_hand_over(self) -> None:
        if getattr(self.worker, "dp", 1) <= 1 or not getattr(self.args, "dp_migration", True):
            return
        from ..runtime.scheduler import plan_cohort_handover
        now = time.monotonic()
        for ticket in [t for t, v in self._handover.items() if now - v[2] > 60.0]:
            del self._handover[ticket]                            # the source never answered: stop waiting for it
        busy = [c for v in self._handover.values() for c in v[:2]]
        plan = plan_cohort_handover(self._cohort_stats, busy)
        if plan is not None:
            self.hand_over(*plan)

    def hand_over(self, src: int, dst: int, rows: int) -> str:
        """Ask cohort ``src`` to pack up to ``rows`` parked rows; they go to ``dst`` when the reply arrives."""
        ticket = uuid.uuid4().hex[:12]
        self._handover[ticket] = (src, dst, time.monotonic())
        self._cohort_stats.get(src, {})["parked"] = 0            # until the next heartbeat says otherwise
        self.worker.send({"type": "migrate_out", "count": rows, "dir": self._handover_dir(), "ticket": ticket, "dst": dst},
                         cohort=src)
        return ticket

    def _on_migrated_out(self, m: Dict[str, Any]) -> None:
        src, dst = self._handover.pop(m.get("ticket"), (int(m.get("cohort", 0)), m.get("dst"), 0.0))[:2]
        rows = m.get("rows") or []
        if not rows or dst is None:
            return
        for row in rows:                                           # the rows' prefill cost now counts for the new cohort
            slot = row["meta"]["slot"]
            done = self._slot_cost.get(slot)
            if done is not None:
                self._dp_load[done[0]] = max(0, self._dp_load[done[0]] - done[1])
                self._dp_load[dst] += done[1]
                self._slot_cost[slot] = (dst, done[1])
        self.migrated_rows += len(rows)
        st = self._cohort_stats.setdefault(dst, {"parked": 0, "live": 0, "host_free": 0})
        st["live"] = st.get("live", 0) + len(rows)
        self.worker.send({"type": "migrate_in", "rows": rows}, cohort=dst)

    def _on_completion(self, m: Dict[str, Any]) -> None:
        done = self._slot_cost.pop(m.get("slot"), None)
        if done is not None:
            self._dp_load[done[0]] = max(0, self._dp_load[done[0]] - done[1])
        bid, rid = m["batch_id"], m["request_id"]
        waiter = self._turn_waiters.get(bid)
        if waiter is not None:
            self.pool.record_request_result(bid, rid, True)
            waiter.put(m)
            return
        with self._lock:
            req = self._reqs.get(bid, {}).get(rid)
            opts = self._opts.get(bid)
        if req is None:
            return
        fr = m.get("finish_reason") or ""
        if fr.startswith("error"):
            item, ok = batch_api.error_item(req, fr, "engine_error"), False
        elif fr == "cancelled":
            item, ok = batch_api.error_item(req, "batch cancelled while the request was running", "cancelled"), False
        else:
            seq = Sequence(global_idx=0, prompt_ids=[0] * m["prompt_tokens"], output_ids=list(m["output_ids"]))
            seq.finish_reason, seq.cached_prefix_tokens = fr, m.get("cached_tokens", 0)
            item, ok = batch_api.result_item(seq, req, self.tok, opts), True
        self._record(bid, rid, item, ok)

    def _record(self, bid: str, rid: str, item: Dict[str, Any], ok: bool) -> None:
        counted, finished = self.pool.record_request_result(bid, rid, ok)
        if not counted:
            return
        self.storage.append_output(bid, item)
        b = self.storage.get_batch(bid)
        if b is None:
            return
        t = self.pool.trackers[bid]
        b.request_counts.completed, b.request_counts.failed = t.completed, t.failed
        if finished and b.status in ("in_progress", "validating", "cancelling"):
            b.status = "finalizing"
            b.finalizing_at = int(time.time())
            fo = self.storage.publish_output(bid)
            b.output_file_id = fo.id if fo else None
            if t.cancelled:
                b.status, b.cancelled_at = "cancelled", int(time.time())
            else:
                b.status, b.completed_at = "completed", int(time.time())
            with self._lock:
                self._reqs.pop(bid, None)
                self._opts.pop(bid, None)
        self.storage.save_batch(b)

    # ------------------------------------------------------------------ cancel / failure
    def cancel(self, bid: str) -> Optional[BatchObject]:
        b = self.storage.get_batch(bid)
        if b is None or b.status not in ("validating", "in_progress"):
            return b
        t = self.pool.trackers.get(bid)
        if t is not None:
            t.cancelled = True
        dropped = self.intake.cancel_batch(bid)
        self.worker.send({"type": "cancel", "batch_id": bid})
        b.status, b.cancelling_at = "cancelling", int(time.time())
        self.storage.save_batch(b)
        with self._lock:
            reqs = dict(self._reqs.get(bid, {}))
        in_flight = {r.request_id for r in self.pool.in_flight(bid)}
        for rid, req in reqs.items():
            if t is not None and rid not in t.done and rid not in in_flight:
                self._record(bid, rid, batch_api.error_item(req, "batch cancelled before the request ran", "cancelled"),
                             ok=False)
        return self.storage.get_batch(bid)

    def fail_in_flight(self, reason: str) -> None:
        """Workers are gone: every batch with requests on the workers fails with the reason; results already
        written stay in its output file."""
        for bid, t in list(self.pool.trackers.items()):
            if t.finished:
                continue
            b = self.storage.get_batch(bid)
            self.intake.cancel_batch(bid)
            self.pool.release_batch(bid)
            if b is not None and b.status in ("validating", "in_progress", "cancelling"):
                self._fail_batch(b, "worker_failure", reason)
            w = self._turn_waiters.get(bid)
            if w is not None:
                w.put({"type": "completion", "finish_reason": f"error: {reason}", "output_ids": [], "prompt_tokens": 0})

    # ------------------------------------------------------------------ synchronous single request (sessions)
    def end_session(self, session_id: str) -> None:
        """Tell the workers that a session is over: its pinned frontier pages become ordinary cache entries."""
        if self.worker.state == "ready":
            self._session_cohort.pop(session_id, None)
            self.worker.send({"type": "end_session", "session_id": session_id})

    def submit_turn(self, prompt_ids: List[int], sampling: Dict[str, Any], timeout: float = 600.0,
                    session_id: Optional[str] = None) -> Dict[str, Any]:
        bid = "turn-" + uuid.uuid4().hex[:16]
        q: "queue_mod.Queue" = queue_mod.Queue()
        self._turn_waiters[bid] = q
        self.pool.register_batch(bid, 1)
        try:
            self.intake.submit_batch([IntakeRequest(bid, "turn", list(prompt_ids), dict(sampling), NORMAL,
                                                    meta={"session_id": session_id})])
            return q.get(timeout=timeout)
        finally:
            self._turn_waiters.pop(bid, None)
            self.pool.trackers.pop(bid, None)
