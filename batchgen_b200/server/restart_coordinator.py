"""Coordinated worker-pool restart and peer liveness across the nodes of one server.

A worker cohort is one ``torch.distributed`` world spanning every node, so no node can replace its ranks
alone: survivors would stay blocked in the old world's collectives while the fresh ranks wait at a rendezvous
nobody joins.  Every node therefore runs the same phase protocol against a small key-value store hosted by
node 0 and leaves a phase only when every node has acknowledged it (or one has reported failure).

The store also carries liveness: each node beats ``alive/<node> = <incarnation>:<beat>``; a watcher follows
the first incarnation it sees for a peer, so a peer whose key is later written by another incarnation has
lost its old process (its cohort died with it), however quickly the new process started beating.  Silence
for longer than ``liveness_timeout_s`` and explicit ``down/<generation>/<node>`` keys are the other two
signals.  A single-node server creates no store and every call returns at once; only the epoch is counted.

The store is anything with ``set(key, str)``, ``get(key) -> str | None`` and ``add(key, n) -> int``
(``InMemoryStore`` here, ``TcpStoreAdapter`` over ``torch.distributed.TCPStore`` across nodes).

Reference parity: batchgen/server/restart_coordinator.py:113-245 (keys, errors, request), :485-660 (begin,
barrier, fail_phase, peer_failed, publish_down), :704-790 (liveness by incarnation, heartbeat).
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

PHASES = ("quiesce", "teardown", "spawn", "ready")


class PeerRestartError(RuntimeError):
    def __init__(self, node: int, phase: str, reason: str):
        super().__init__(f"node {node} failed restart phase {phase!r}: {reason}")
        self.node, self.phase, self.reason = node, phase, reason


class RestartTimeout(RuntimeError):
    pass


class InMemoryStore:
    def __init__(self):
        self._d: Dict[str, str] = {}
        self._mu = threading.Lock()

    def set(self, key: str, value: str) -> None:
        with self._mu:
            self._d[key] = str(value)

    def get(self, key: str) -> Optional[str]:
        with self._mu:
            return self._d.get(key)

    def add(self, key: str, n: int) -> int:
        with self._mu:
            v = int(self._d.get(key, "0")) + n
            self._d[key] = str(v)
            return v


class TcpStoreAdapter:
    """``torch.distributed.TCPStore`` behind the same three calls (``get`` of a missing key returns None)."""

    def __init__(self, host: str, port: int, is_master: bool, timeout_s: float = 30.0):
        import datetime
        from torch.distributed import TCPStore
        self._s = TCPStore(host, port, is_master=is_master, timeout=datetime.timedelta(seconds=timeout_s),
                           wait_for_workers=False)

    def set(self, key: str, value: str) -> None:
        self._s.set(key, value)

    def get(self, key: str) -> Optional[str]:
        if not self._s.check([key]):
            return None
        return self._s.get(key).decode()

    def add(self, key: str, n: int) -> int:
        return int(self._s.add(key, n))


@dataclass(frozen=True)
class RestartRequest:
    epoch: int
    issued_at: float
    timeout_s: float

    @property
    def deadline(self) -> float:
        return self.issued_at + self.timeout_s


class RestartCoordinator:
    def __init__(self, node_rank: int, nnodes: int, store: Any = None, heartbeat_s: float = 0.5,
                 liveness_timeout_s: float = 5.0, clock: Callable[[], float] = time.monotonic):
        self.node_rank, self.nnodes = node_rank, nnodes
        self.store = store if nnodes > 1 else None
        if nnodes > 1 and store is None:
            raise ValueError("a multi-node server needs a control store")
        self.heartbeat_s, self.liveness_timeout_s, self._clock = heartbeat_s, liveness_timeout_s, clock
        self.incarnation = uuid.uuid4().hex[:12]
        self._epoch = 0
        self._beat = 0
        self._seen: Dict[int, Tuple[str, int, float]] = {}      # node -> (incarnation, last beat, when it changed)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    @property
    def enabled(self) -> bool:
        return self.store is not None

    @property
    def epoch(self) -> int:
        return self._epoch

    # ------------------------------------------------------------------ restart phases
    def begin_restart(self, timeout_s: float) -> RestartRequest:
        """Node 0 only: open a new epoch and publish the request."""
        if self.node_rank != 0:
            raise RuntimeError("only node 0 opens a restart epoch")
        if not self.enabled:
            self._epoch += 1
            return RestartRequest(self._epoch, self._clock(), timeout_s)
        self._epoch = self.store.add("restart/epoch", 1)
        req = RestartRequest(self._epoch, self._clock(), timeout_s)
        self.store.set(f"restart/{req.epoch}/request", json.dumps({"timeout_s": timeout_s}))
        return req

    def poll_request(self) -> Optional[RestartRequest]:
        """Followers: a request for an epoch newer than the one this node last ran, if any."""
        if not self.enabled:
            return None
        cur = int(self.store.get("restart/epoch") or 0)
        if cur <= self._epoch:
            return None
        raw = self.store.get(f"restart/{cur}/request")
        if raw is None:
            return None
        self._epoch = cur
        return RestartRequest(cur, self._clock(), float(json.loads(raw)["timeout_s"]))

    def barrier(self, epoch: int, phase: str, deadline: float, poll_s: float = 0.01) -> None:
        """Acknowledge ``phase`` and wait until every node has, a peer failed, or the deadline passes."""
        if not self.enabled:
            return
        self.store.set(f"restart/{epoch}/{phase}/{self.node_rank}", "ok")
        while True:
            missing = []
            for n in range(self.nnodes):
                v = self.store.get(f"restart/{epoch}/{phase}/{n}")
                if v is None:
                    missing.append(n)
                elif v != "ok":
                    raise PeerRestartError(n, phase, v[len("failed:"):] if v.startswith("failed:") else v)
            if not missing:
                return
            if self._clock() > deadline:
                raise RestartTimeout(f"restart epoch {epoch} phase {phase!r}: no acknowledgement from nodes {missing}")
            time.sleep(poll_s)

    def fail_phase(self, epoch: int, phase: str, reason: str) -> None:
        if self.enabled:
            self.store.set(f"restart/{epoch}/{phase}/{self.node_rank}", "failed:" + reason[:200])

    def publish_result(self, epoch: int, result: Dict[str, Any]) -> None:
        if self.enabled:
            self.store.set(f"restart/{epoch}/result", json.dumps(result))

    def run_phases(self, req: RestartRequest, hooks: Dict[str, Callable[[], None]]) -> None:
        """The same function on every node: run each phase's hook, then meet the others."""
        for phase in PHASES:
            try:
                hooks.get(phase, lambda: None)()
            except Exception as exc:                      # noqa: BLE001 - reported to the peers by name
                self.fail_phase(req.epoch, phase, repr(exc))
                raise
            self.barrier(req.epoch, phase, req.deadline)

    # ------------------------------------------------------------------ liveness
    def publish_down(self, generation: int, reason: str) -> None:
        if self.enabled:
            self.store.set(f"down/{generation}/{self.node_rank}", reason[:200])

    def beat(self) -> None:
        if self.enabled:
            self._beat += 1
            self.store.set(f"alive/{self.node_rank}", f"{self.incarnation}:{self._beat}")

    def check_peers(self, generation: int = 0) -> Optional[Tuple[int, str]]:
        """(node, reason) for the first peer that is down, replaced by another process, or silent too long."""
        if not self.enabled:
            return None
        now = self._clock()
        for n in range(self.nnodes):
            if n == self.node_rank:
                continue
            down = self.store.get(f"down/{generation}/{n}")
            if down is not None:
                return n, f"reported down: {down}"
            raw = self.store.get(f"alive/{n}")
            if raw is None:
                first = self._seen.setdefault(n, ("", -1, now))
                if now - first[2] > self.liveness_timeout_s:
                    return n, "never started beating"
                continue
            inc, beat = raw.rsplit(":", 1)
            prev = self._seen.get(n)
            if prev is None or prev[0] == "":
                self._seen[n] = (inc, int(beat), now)
            elif prev[0] != inc:
                return n, f"process replaced (incarnation {prev[0]} -> {inc})"
            elif int(beat) != prev[1]:
                self._seen[n] = (inc, int(beat), now)
            elif now - prev[2] > self.liveness_timeout_s:
                return n, f"silent for {now - prev[2]:.1f} s"
        return None

    def start(self, on_peer_lost: Optional[Callable[[int, str], None]] = None) -> None:
        if not self.enabled or self._thread is not None:
            return

        def loop():
            while not self._stop.wait(self.heartbeat_s):
                self.beat()
                lost = self.check_peers()
                if lost is not None and on_peer_lost is not None:
                    on_peer_lost(*lost)
                    return

        self.beat()
        self._thread = threading.Thread(target=loop, name="bg-restart-heartbeat", daemon=True)
        self._thread.start()

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None
