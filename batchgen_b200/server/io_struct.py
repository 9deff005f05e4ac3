"""OpenAI-compatible request / response models of the HTTP API (pydantic).

Shapes follow docs/batch-api.md and batchgen/server/io_struct.py of the reference: ``FileObject``,
``BatchObject`` (status flow ``validating -> in_progress -> completed | failed | cancelled``, live
``request_counts``), ``CreateBatchRequest`` with the engine extensions (``max_decoding_length``,
per-batch sampling defaults, ``batchgen_debug``), session / turn bodies, worker and pool status.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Literal, Optional

from pydantic import BaseModel, Field

BatchStatus = Literal["validating", "in_progress", "finalizing", "completed", "failed", "cancelling", "cancelled",
                      "expired"]


def new_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


class FileObject(BaseModel):
    id: str = Field(default_factory=lambda: new_id("file"))
    object: str = "file"
    bytes: int = 0
    created_at: int = Field(default_factory=lambda: int(time.time()))
    filename: str = ""
    purpose: str = "batch"
    sha256: Optional[str] = None


class FileList(BaseModel):
    object: str = "list"
    data: List[FileObject] = []


class FileDeleted(BaseModel):
    id: str
    object: str = "file"
    deleted: bool = True


class RequestCounts(BaseModel):
    total: int = 0
    completed: int = 0
    failed: int = 0


class BatchError(BaseModel):
    code: str = "invalid_request"
    message: str = ""
    line: Optional[int] = None


class BatchErrors(BaseModel):
    object: str = "list"
    data: List[BatchError] = []


class CreateBatchRequest(BaseModel):
    input_file_id: str
    endpoint: Literal["/v1/chat/completions", "/v1/completions"] = "/v1/chat/completions"
    completion_window: str = "24h"
    metadata: Optional[Dict[str, str]] = None
    # engine extensions
    max_decoding_length: Optional[int] = Field(default=None, gt=0)
    temperature: Optional[float] = Field(default=None, ge=0)
    top_p: Optional[float] = Field(default=None, gt=0, le=1)
    top_k: Optional[int] = Field(default=None, ge=0)
    batchgen_debug: Optional[Dict[str, Any]] = None


class BatchObject(BaseModel):
    id: str = Field(default_factory=lambda: new_id("batch"))
    object: str = "batch"
    endpoint: str = "/v1/chat/completions"
    errors: Optional[BatchErrors] = None
    input_file_id: str = ""
    completion_window: str = "24h"
    status: BatchStatus = "validating"
    output_file_id: Optional[str] = None
    error_file_id: Optional[str] = None
    created_at: int = Field(default_factory=lambda: int(time.time()))
    in_progress_at: Optional[int] = None
    finalizing_at: Optional[int] = None
    completed_at: Optional[int] = None
    failed_at: Optional[int] = None
    cancelling_at: Optional[int] = None
    cancelled_at: Optional[int] = None
    request_counts: RequestCounts = RequestCounts()
    metadata: Optional[Dict[str, str]] = None
    max_decoding_length: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    batchgen_debug: Optional[Dict[str, Any]] = None


class BatchList(BaseModel):
    object: str = "list"
    data: List[BatchObject] = []
    has_more: bool = False


class ModelCard(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "batchgen_b200"
    max_model_len: Optional[int] = None


class ModelList(BaseModel):
    object: str = "list"
    data: List[ModelCard] = []


class CreateSessionRequest(BaseModel):
    metadata: Optional[Dict[str, str]] = None


class SessionObject(BaseModel):
    id: str = Field(default_factory=lambda: new_id("sess"))
    object: str = "session"
    status: Literal["open", "closed", "aborted"] = "open"
    created_at: int = Field(default_factory=lambda: int(time.time()))
    turns: int = 0
    context_tokens: int = 0
    metadata: Optional[Dict[str, str]] = None


class TurnRequest(BaseModel):
    session_id: str
    messages: Optional[List[Dict[str, Any]]] = None
    prompt: Optional[Any] = None
    max_completion_tokens: Optional[int] = Field(default=None, gt=0)
    max_tokens: Optional[int] = Field(default=None, gt=0)
    temperature: Optional[float] = Field(default=None, ge=0)
    top_p: Optional[float] = Field(default=None, gt=0, le=1)
    top_k: Optional[int] = Field(default=None, ge=0)
    ignore_eos: bool = False


class TurnResponse(BaseModel):
    id: str = Field(default_factory=lambda: new_id("turn"))
    object: str = "turn"
    session_id: str = ""
    turn_index: int = 0
    choices: List[Dict[str, Any]] = []
    usage: Dict[str, Any] = {}


class WorkerStatus(BaseModel):
    state: str = "stopped"                 # stopped | starting | ready | restarting | failed
    generation: int = 0
    world_size: int = 0
    pids: List[int] = []
    last_error: Optional[str] = None
    capacity: Optional[Dict[str, Any]] = None


class PoolStatus(BaseModel):
    serving: bool = False
    intake_size: int = 0
    intake_capacity: int = 0
    scheduling_slots_total: int = 0
    scheduling_slots_used: int = 0
    batches_in_flight: int = 0


class HealthResponse(BaseModel):
    status: str = "starting"               # starting | ok | degraded | failed
    startup_complete: bool = False
    workers: str = "stopped"
    detail: Optional[str] = None
