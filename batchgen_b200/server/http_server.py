"""OpenAI-style file / batch HTTP server.

Routes: ``GET /v1/models[/{id}]``; ``POST/GET /v1/files``, ``GET/DELETE /v1/files/{id}``,
``GET /v1/files/{id}/content``; ``POST/GET /v1/batches``, ``GET /v1/batches/{id}``,
``POST /v1/batches/{id}/cancel``; ``POST /v1/sessions``, ``POST /v1/sessions/{id}/close|abort``,
``GET /v1/sessions/{id}``, ``POST /v1/turns``; ``POST /v1/workers/restart``, ``GET /v1/workers/status``;
``GET /v1/pool/status``; ``GET /health``; ``POST /v1/inference`` answers 410 (the legacy synchronous API is
gone).  While the worker pool is not serving, batch creation answers 503 with ``Retry-After``; when the intake
pool is more than 90 % full it answers 429.

Reference parity: batchgen/server/http_server.py:178-732 (app, lifespan wiring :187-259, routes :305-730,
gates :474-498), batchgen/server/turn_api.py + agent_sessions.py (session state machine), docs/batch-api.md.
"""
from __future__ import annotations

import threading
import time
from contextlib import asynccontextmanager
from typing import Dict, Optional

from fastapi import FastAPI, File, Form, HTTPException, Response, UploadFile
from fastapi.responses import JSONResponse, PlainTextResponse

from ..config import get_model_config
from ..runtime import batch_api
from ..runtime.tokenization import chat_format_for, get_tokenizer
from .batch_scheduler import BatchScheduler
from .io_struct import (BatchList, BatchObject, CreateBatchRequest, CreateSessionRequest, FileDeleted, FileList,
                        HealthResponse, ModelCard, ModelList, PoolStatus, SessionObject, TurnRequest, TurnResponse)
from .server_args import ServerArgs
from .storage import StorageManager
from .worker_manager import WorkerManager, WorkerStartError


class ServerHealthState:
    def __init__(self):
        self.startup_complete = False
        self.detail: Optional[str] = None

    def mark_startup_complete(self) -> None:
        self.startup_complete = True


class SessionStore:
    """Agent sessions: a growing token context per session; each turn extends it.  With the prefix cache
    on, a turn's prompt re-uses the pages its predecessors committed, so only the new tokens are computed
    (the reference restores a committed "trajectory frontier": batchgen/prefix_reuse/trajectory_frontier.py)."""

    def __init__(self):
        self.sessions: Dict[str, SessionObject] = {}
        self.context: Dict[str, list] = {}
        self.tombstones: Dict[str, str] = {}
        self._lock = threading.Lock()

    def create(self, meta) -> SessionObject:
        s = SessionObject(metadata=meta)
        with self._lock:
            self.sessions[s.id] = s
            self.context[s.id] = []
        return s

    def get(self, sid: str) -> SessionObject:
        s = self.sessions.get(sid)
        if s is None:
            if sid in self.tombstones:
                raise HTTPException(410, f"session {sid} was {self.tombstones[sid]}")
            raise HTTPException(404, f"no session {sid}")
        return s

    def end(self, sid: str, how: str) -> SessionObject:
        s = self.get(sid)
        with self._lock:
            s.status = how
            self.tombstones[sid] = how
            self.sessions.pop(sid, None)
            self.context.pop(sid, None)
        return s


def create_app(args: ServerArgs, worker: Optional[WorkerManager] = None, start_workers: bool = True) -> FastAPI:
    cfg = get_model_config(args.model)
    storage = StorageManager(args.storage_path)
    worker = worker or WorkerManager(args)
    tokenizer = get_tokenizer(args.tokenizer, cfg.vocab_size, cfg.bos_token_id, cfg.eos_token_id,
                              chat_format=chat_format_for(cfg.family))
    scheduler = BatchScheduler(storage, worker, args, tokenizer)
    health = ServerHealthState()
    sessions = SessionStore()

    @asynccontextmanager
    async def lifespan(app: FastAPI):
        storage.acquire_ownership()
        orphans = storage.fail_orphaned_batches()
        worker.set_lifecycle_hooks(quiesce=scheduler.quiesce, resume=scheduler.resume,
                                   fail_in_flight=scheduler.fail_in_flight, has_work=scheduler.has_work,
                                   rebind_queues=scheduler.rebind_queues)
        scheduler.start()
        if start_workers:
            try:
                worker.start()
            except WorkerStartError as e:
                health.detail = str(e)
        health.mark_startup_complete()
        app.state.orphans = orphans
        try:
            yield
        finally:
            scheduler.stop()
            worker.stop()
            storage.release_ownership()

    app = FastAPI(title="batchgen_b200", lifespan=lifespan)
    app.state.storage, app.state.worker, app.state.scheduler = storage, worker, scheduler
    app.state.health, app.state.sessions, app.state.args = health, sessions, args

    # ------------------------------------------------------------------ models
    @app.get("/v1/models")
    def list_models_route() -> ModelList:
        return ModelList(data=[ModelCard(id=args.model, max_model_len=(scheduler.capacity or {}).get("kv_token_budget"))])

    @app.get("/v1/models/{model_id:path}")
    def get_model(model_id: str) -> ModelCard:
        if model_id != args.model:
            raise HTTPException(404, f"model {model_id} is not served")
        return ModelCard(id=args.model, max_model_len=(scheduler.capacity or {}).get("kv_token_budget"))

    # ------------------------------------------------------------------ files
    @app.post("/v1/files")
    async def upload_file(file: UploadFile = File(...), purpose: str = Form("batch")):
        data = await file.read()
        if purpose == "batch":
            try:
                batch_api.parse_batch_lines(data.decode("utf-8", errors="replace").splitlines(), None)
            except batch_api.BatchFormatError as e:
                raise HTTPException(400, f"invalid batch file: {e}")
        return storage.save_file(data, file.filename or "upload.jsonl", purpose)

    @app.get("/v1/files")
    def list_files() -> FileList:
        return FileList(data=storage.list_files())

    @app.get("/v1/files/{file_id}")
    def get_file(file_id: str):
        f = storage.get_file(file_id)
        if f is None:
            raise HTTPException(404, f"no file {file_id}")
        return f

    @app.delete("/v1/files/{file_id}")
    def delete_file(file_id: str) -> FileDeleted:
        if not storage.delete_file(file_id):
            raise HTTPException(404, f"no file {file_id}")
        return FileDeleted(id=file_id)

    @app.get("/v1/files/{file_id}/content")
    def file_content(file_id: str):
        data = storage.read_file(file_id)
        if data is None:
            raise HTTPException(404, f"no file {file_id}")
        return PlainTextResponse(data.decode("utf-8", errors="replace"), media_type="application/jsonl")

    # ------------------------------------------------------------------ batches
    @app.post("/v1/batches")
    def create_batch(req: CreateBatchRequest):
        if worker.state != "ready":
            return JSONResponse({"error": {"message": f"worker pool is {worker.state}", "type": "pool_not_serving"}},
                                status_code=503, headers={"Retry-After": "5"})
        if scheduler.intake.fill_fraction > 0.9:
            return JSONResponse({"error": {"message": "intake pool above 90 %", "type": "intake_full"}},
                                status_code=429, headers={"Retry-After": "10"})
        if storage.get_file(req.input_file_id) is None:
            raise HTTPException(404, f"no file {req.input_file_id}")
        b = BatchObject(endpoint=req.endpoint, input_file_id=req.input_file_id, completion_window=req.completion_window,
                        metadata=req.metadata, max_decoding_length=req.max_decoding_length, temperature=req.temperature,
                        top_p=req.top_p, top_k=req.top_k, batchgen_debug=req.batchgen_debug)
        storage.save_batch(b)
        scheduler.enqueue(b)
        return b

    @app.get("/v1/batches")
    def list_batches(limit: int = 100) -> BatchList:
        bs = storage.list_batches()
        return BatchList(data=bs[-limit:], has_more=len(bs) > limit)

    @app.get("/v1/batches/{batch_id}")
    def get_batch(batch_id: str):
        b = storage.get_batch(batch_id)
        if b is None:
            raise HTTPException(404, f"no batch {batch_id}")
        return b

    @app.post("/v1/batches/{batch_id}/cancel")
    def cancel_batch(batch_id: str):
        b = scheduler.cancel(batch_id)
        if b is None:
            raise HTTPException(404, f"no batch {batch_id}")
        return b

    # ------------------------------------------------------------------ sessions / turns
    @app.post("/v1/sessions")
    def create_session(req: CreateSessionRequest) -> SessionObject:
        return sessions.create(req.metadata)

    @app.get("/v1/sessions/{sid}")
    def get_session(sid: str) -> SessionObject:
        return sessions.get(sid)

    @app.post("/v1/sessions/{sid}/close")
    def close_session(sid: str) -> SessionObject:
        out = sessions.end(sid, "closed")
        scheduler.end_session(sid)
        return out

    @app.post("/v1/sessions/{sid}/abort")
    def abort_session(sid: str) -> SessionObject:
        out = sessions.end(sid, "aborted")
        scheduler.end_session(sid)
        return out

    @app.post("/v1/turns")
    def turn(req: TurnRequest) -> TurnResponse:
        s = sessions.get(req.session_id)
        if worker.state != "ready":
            raise HTTPException(503, f"worker pool is {worker.state}")
        if req.messages is not None:
            new_ids = list(tokenizer.apply_chat_template(req.messages, add_generation_prompt=True))
        elif req.prompt is not None:
            new_ids = list(tokenizer.encode(req.prompt))
        else:
            raise HTTPException(400, "a turn needs messages or prompt")
        ctx = sessions.context[s.id]
        prompt = ctx + new_ids
        sampling = dict(temperature=req.temperature or 0.0, top_p=req.top_p or 1.0, top_k=req.top_k or 0,
                        max_new_tokens=req.max_completion_tokens or req.max_tokens or 256, ignore_eos=req.ignore_eos,
                        seed=None)
        m = scheduler.submit_turn(prompt, sampling, session_id=s.id)
        fr = m.get("finish_reason") or ""
        if fr.startswith("error"):
            raise HTTPException(500, fr)
        out = list(m["output_ids"])
        sessions.context[s.id] = prompt + out
        s.turns += 1
        s.context_tokens = len(prompt) + len(out)
        text = tokenizer.decode(out)
        return TurnResponse(session_id=s.id, turn_index=s.turns - 1,
                            choices=[{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": fr}],
                            usage={"prompt_tokens": len(prompt), "completion_tokens": len(out),
                                   "total_tokens": len(prompt) + len(out),
                                   "prompt_tokens_details": {"cached_tokens": m.get("cached_tokens", 0)}})

    # ------------------------------------------------------------------ control
    @app.post("/v1/workers/restart")
    def restart_workers():
        try:
            gen = worker.restart_workers("POST /v1/workers/restart")
        except WorkerStartError as e:
            raise HTTPException(500, str(e))
        return {"status": "restarted", "generation": gen}

    @app.get("/v1/workers/status")
    def workers_status():
        st = dict(worker.status())
        beat = scheduler.last_heartbeat
        if beat:                         # engine counters, recent steps and memory of the worker's last heartbeat
            st["heartbeat"] = {k: beat.get(k) for k in ("ts", "live", "free_pages", "stats", "steps", "memory", "query_book")}
        return st

    @app.get("/v1/pool/status")
    def pool_status() -> PoolStatus:
        return PoolStatus(serving=worker.state == "ready", intake_size=len(scheduler.intake),
                          intake_capacity=scheduler.intake.capacity, scheduling_slots_total=scheduler.pool.slots,
                          scheduling_slots_used=scheduler.pool.used,
                          batches_in_flight=sum(1 for t in scheduler.pool.trackers.values() if not t.finished))

    @app.get("/health")
    def health_route():
        st = "ok" if (health.startup_complete and worker.state == "ready") else (
            "failed" if worker.state == "failed" else "starting")
        detail = health.detail or worker.last_error
        if st == "starting" and not detail and getattr(worker, "startup", None) is not None:
            try:                                   # where every worker is in its start-up: "worker 0: model-build (12 s)"
                snap = worker.startup.snapshot()
                detail = "; ".join(f"worker {k}: {p} ({int(t)} s)" for k, (p, t) in sorted(snap.items())) or None
            except Exception:  # noqa: BLE001 - the record may be gone while the cohort is being replaced
                detail = None
        body = HealthResponse(status=st, startup_complete=health.startup_complete, workers=worker.state, detail=detail)
        return JSONResponse(body.model_dump(), status_code=200 if st == "ok" else 503)

    @app.post("/v1/inference")
    def legacy_inference():
        return JSONResponse({"error": {"message": "the synchronous /v1/inference API was removed; use /v1/files + "
                                                  "/v1/batches", "type": "gone"}}, status_code=410)

    return app


def launch_server(args: ServerArgs) -> None:
    """Blocking: serve until interrupted.  A start-up watchdog ends the process if the server has not
    finished start-up within ``--startup-timeout``."""
    import os
    import signal

    import uvicorn

    app = create_app(args)

    def startup_watchdog():
        deadline = time.monotonic() + args.startup_timeout
        while time.monotonic() < deadline:
            if app.state.health.startup_complete:
                return
            time.sleep(1.0)
        os._exit(3)

    threading.Thread(target=startup_watchdog, name="startup-watchdog", daemon=True).start()
    for sig in (signal.SIGTERM, signal.SIGQUIT):
        signal.signal(sig, lambda *_: (_ for _ in ()).throw(KeyboardInterrupt()))
    uvicorn.run(app, host=args.host, port=args.port, log_level="warning", access_log=False)
