"""Structured event log: one JSONL file per process, a console renderer, a crash-surviving flight
recorder and rate-limited step counters.

Every record is a schema-v1 envelope ``{"v": 1, "ts": ..., "proc": ..., "pid": ..., "level": ...,
"event": ..., "batch_id": ..., "fields": {...}}``.  Producers never block on disk: records go through a
queue to a listener thread.  The flight recorder is a fixed-size ring *file* written with ``os.pwrite``
at record time (no buffering), so the last N records of a process survive SIGKILL.

Reference parity: batchgen/eventlog/{schema,handlers,process,flight_recorder,counters,context,console}.py
(schema v1 envelope schema.py:24-52, flight recorder flight_recorder.py:1-40, step counters
counters.py:14-60).
"""
from __future__ import annotations

import contextlib
import contextvars
import json
import os
import queue
import sys
import threading
import time
from typing import Any, Dict, Optional

SCHEMA_VERSION = 1
LEVELS = {"debug": 10, "info": 20, "warning": 30, "error": 40, "fatal": 50}
_batch_ctx: contextvars.ContextVar = contextvars.ContextVar("bg_batch_id", default=None)


def make_record(proc: str, level: str, event: str, fields: Optional[Dict[str, Any]] = None,
                batch_id: Optional[str] = None) -> Dict[str, Any]:
    if level not in LEVELS:
        raise ValueError(f"unknown level {level!r}")
    return {"v": SCHEMA_VERSION, "ts": time.time(), "proc": proc, "pid": os.getpid(), "level": level,
            "event": event, "batch_id": batch_id if batch_id is not None else _batch_ctx.get(),
            "fields": fields or {}}


def validate_record(rec: Dict[str, Any]) -> None:
    for k in ("v", "ts", "proc", "pid", "level", "event", "fields"):
        if k not in rec:
            raise ValueError(f"record lacks {k!r}")
    if rec["v"] != SCHEMA_VERSION or rec["level"] not in LEVELS or not isinstance(rec["fields"], dict):
        raise ValueError("malformed record")


@contextlib.contextmanager
def batch_context(batch_id: str):
    tok = _batch_ctx.set(batch_id)
    try:
        yield
    finally:
        _batch_ctx.reset(tok)


class FlightRecorder:
    """Ring file of ``slots`` fixed-size records; readable after the writer was killed."""

    def __init__(self, path: str, slots: int = 256, slot_bytes: int = 512):
        self.path, self.slots, self.slot_bytes = path, slots, slot_bytes
        self._fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o644)
        os.ftruncate(self._fd, slots * slot_bytes)
        self._n = 0
        self._lock = threading.Lock()

    def record(self, rec: Dict[str, Any]) -> None:
        with self._lock:
            seq = self._n
            self._n += 1
        body = json.dumps({"seq": seq, **rec}, default=str).encode()[: self.slot_bytes - 1]
        os.pwrite(self._fd, body.ljust(self.slot_bytes - 1, b" ") + b"\n", (seq % self.slots) * self.slot_bytes)

    def close(self) -> None:
        os.close(self._fd)

    @staticmethod
    def read(path: str, slot_bytes: int = 512):
        out = []
        with open(path, "rb") as f:
            data = f.read()
        for i in range(0, len(data), slot_bytes):
            chunk = data[i:i + slot_bytes].strip(b"\x00 \n")
            if not chunk:
                continue
            try:
                out.append(json.loads(chunk))
            except ValueError:
                continue        # a record that was truncated to the slot size
        return sorted(out, key=lambda r: r.get("seq", 0))


class EventLog:
    def __init__(self, proc: str, log_dir: Optional[str] = None, level: str = "info", console: bool = False,
                 flight_recorder: bool = False):
        self.proc, self.level = proc, LEVELS[level]
        self.console = console
        self._q: "queue.Queue" = queue.Queue()
        self._file = None
        self.path = None
        self.flight: Optional[FlightRecorder] = None
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)
            self.path = os.path.join(log_dir, f"{proc}.{os.getpid()}.jsonl")
            self._file = open(self.path, "a", buffering=1)
            if flight_recorder:
                self.flight = FlightRecorder(os.path.join(log_dir, f"{proc}.{os.getpid()}.flight"))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._listen, name=f"eventlog-{proc}", daemon=True)
        self._thread.start()

    def _listen(self) -> None:
        while True:
            rec = self._q.get()
            if rec is None:
                break
            line = json.dumps(rec, default=str)
            if self._file is not None:
                self._file.write(line + "\n")
            if self.console:
                f = rec["fields"]
                kv = " ".join(f"{k}={v}" for k, v in f.items())
                print(f"[{rec['level'].upper():7s}] {rec['proc']} {rec['event']} {kv}", file=sys.stderr)

    def emit(self, level: str, event: str, **fields) -> None:
        if LEVELS[level] < self.level:
            return
        rec = make_record(self.proc, level, event, fields)
        if self.flight is not None:
            self.flight.record(rec)
        self._q.put(rec)

    def info(self, event: str, **f) -> None:
        self.emit("info", event, **f)

    def warning(self, event: str, **f) -> None:
        self.emit("warning", event, **f)

    def error(self, event: str, **f) -> None:
        self.emit("error", event, **f)

    def close(self) -> None:
        self._q.put(None)
        self._thread.join(timeout=5)
        if self._file is not None:
            self._file.close()
        if self.flight is not None:
            self.flight.close()


class StepCounters:
    """Counters that are cheap to bump every decode step and are logged at most every ``period`` s."""

    def __init__(self, log: Optional[EventLog], period: float = 30.0):
        self.log, self.period = log, period
        self.c: Dict[str, float] = {}
        self._last = time.monotonic()

    def bump(self, name: str, by: float = 1) -> None:
        self.c[name] = self.c.get(name, 0) + by

    def maybe_flush(self, force: bool = False) -> bool:
        now = time.monotonic()
        if not force and now - self._last < self.period:
            return False
        self._last = now
        if self.log is not None:
            self.log.info("step.counters", **self.c)
        return True


_process_log: Optional[EventLog] = None


def configure_process(proc: str, log_dir: Optional[str] = None, level: str = "info", console: bool = False,
                      flight_recorder: bool = False) -> EventLog:
    global _process_log
    if _process_log is not None:
        _process_log.close()
    _process_log = EventLog(proc, log_dir, level, console, flight_recorder)
    return _process_log


def get_log() -> EventLog:
    global _process_log
    if _process_log is None:
        _process_log = EventLog("proc")
    return _process_log
