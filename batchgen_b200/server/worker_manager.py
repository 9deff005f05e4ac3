"""WorkerManager: owns the worker cohort (one process per GPU), its queues, its liveness and its restarts.

``start()`` spawns the cohort (``multiprocessing`` *spawn* context, so CUDA is initialised only in the
children), waits for rank 0's readiness event and starts a monitor thread that notices a dead worker within
a poll period and fails the cohort fast: a lost rank takes the whole generation down (world size is fixed,
as in the reference's cluster fail-fast, docs/server-flags.md:126-146), in-flight batches are failed with the
reason through the lifecycle hooks, and the server keeps its storage.  ``restart_workers()`` replaces the
cohort with a new generation (phases: P0 quiesce intake, P1 stop old cohort, P2 start new cohort and resume),
the equivalent of ``POST /v1/workers/restart``.

Reference parity: batchgen/server/worker_manager.py:177,668 (start), :1433 (restart), :1819-1980 (spawn),
:2062-2250 (exit monitor), batchgen/server/restart_coordinator.py (epochs and phases; single node here, so
the TCPStore control plane reduces to in-process state), batchgen/server/watchdog.py:19-197.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import threading
import time
from typing import Callable, Dict, List, Optional

from .io_struct import WorkerStatus
from .server_args import ServerArgs


class WorkerStartError(RuntimeError):
    pass


class Watchdog(threading.Thread):
    """Feed-counter watchdog: if the counter does not move for ``timeout`` seconds while ``armed()`` is true,
    ``on_stall(elapsed)`` runs once per stall."""

    def __init__(self, read_counter: Callable[[], int], timeout: float, on_stall: Callable[[float], None],
                 armed: Callable[[], bool] = lambda: True, period: float = 0.25):
        super().__init__(name="watchdog", daemon=True)
        self.read, self.timeout, self.on_stall, self.armed, self.period = read_counter, timeout, on_stall, armed, period
        self._stop = threading.Event()
        self.stalls = 0

    def run(self) -> None:
        last, since, fired = self.read(), time.monotonic(), False
        while not self._stop.wait(self.period):
            cur = self.read()
            now = time.monotonic()
            if cur != last or not self.armed():
                last, since, fired = cur, now, False
            elif not fired and now - since > self.timeout:
                fired = True
                self.stalls += 1
                self.on_stall(now - since)

    def stop(self) -> None:
        self._stop.set()


class WorkerManager:
    def __init__(self, args: ServerArgs, worker_target=None):
        self.args = args
        self.ctx = mp.get_context("spawn")
        # data parallelism: dp_size cohorts of world_size / dp_size ranks, each with its own request queue (and its own
        # process group, engine and KV pool); all report on one response queue
        self.dp = max(1, int(getattr(args, "dp_size", 1)))
        self.request_queues = [self.ctx.Queue() for _ in range(self.dp)]
        self.request_queue = self.request_queues[0]
        self.response_queue = self.ctx.Queue()
        self.procs: List[mp.Process] = []
        self.generation = 0
        self.state = "stopped"
        self.last_error: Optional[str] = None
        self.capacity: Optional[Dict] = None
        self._ready_events = [self.ctx.Event() for _ in range(self.dp)]
        self._ready = self._ready_events[0]
        self._shutdown = self.ctx.Event()
        self.feed = self.ctx.Value("q", 0)
        self._monitor: Optional[threading.Thread] = None
        self._monitor_stop = threading.Event()
        self._hooks: Dict[str, Callable] = {}
        self._target = worker_target
        self.host_region = None                           # node-shared host KV region (core.native.HostPagedKV)
        self.weight_store = None                          # node-shared weights (core.native.ParameterStore)
        self.weight_index: Optional[Dict] = None
        self.startup = None                               # server.startup_phases.StartupRecord of the current cohort
        self.startup_budgets: Optional[Dict[str, float]] = None      # None: the module's defaults
        self.kernel_log_path = "/dev/kmsg"
        self._lock = threading.RLock()
        self.watchdog: Optional[Watchdog] = None
        self.phase = "idle"

    # ------------------------------------------------------------------ hooks
    def set_lifecycle_hooks(self, **hooks: Callable) -> None:
        """quiesce(), resume(), fail_in_flight(reason): called around restarts and on cohort loss."""
        self._hooks.update(hooks)

    def _hook(self, name: str, *a) -> None:
        h = self._hooks.get(name)
        if h is not None:
            h(*a)

    def send(self, msg: Dict, cohort: Optional[int] = None) -> None:
        """A message for one cohort, or for all of them (cancel, end of a session, shutdown)."""
        for c in (range(self.dp) if cohort is None else [cohort]):
            self.request_queues[c].put(msg)

    # ------------------------------------------------------------------ start / stop
    def start(self, timeout: Optional[float] = None) -> None:
        with self._lock:
            if self.state in ("starting", "ready"):
                return
            from .worker import worker_main
            target = self._target or worker_main
            self.state = "starting"
            self.generation += 1
            for e in self._ready_events:
                e.clear()
            self._shutdown.clear()
            self.last_error = None
            W = self.args.world_size
            self.procs = []
            from . import startup_phases
            self.startup = startup_phases.StartupRecord(W + 1, self.ctx)    # slot W: the server's own phases
            self.args.startup_record = self.startup
            self._create_host_region()
            with self.startup.phase(W, "store-staging"):
                self._load_weight_store()
            self.startup.enter(W, "serving")
            Wc = W // self.dp
            self.args.param_store_index = self.weight_index      # travels with the pickled arguments
            for c in range(self.dp):
                a = self.args
                if self.dp > 1:                                   # the cohort's own view of the deployment
                    import dataclasses
                    host, port = str(self.args.dist_init_addr).rsplit(":", 1)
                    a = dataclasses.replace(self.args, world_size=Wc, dist_init_addr=f"{host}:{int(port) + c}")
                    for k in ("startup_record", "param_store_index"):
                        setattr(a, k, getattr(self.args, k, None))
                    a.dp_rank, a.gpu_offset, a.startup_slot_base = c, c * Wc, c * Wc
                for r in range(Wc):
                    p = self.ctx.Process(target=target, name=f"bg-worker-{c * Wc + r}",
                                         args=(r, Wc, a, self.request_queues[c], self.response_queue,
                                               self._ready_events[c], self._shutdown, self.feed), daemon=True)
                    p.start()
                    self.startup.enter(c * Wc + r, "spawned")
                    self.procs.append(p)
        deadline = time.monotonic() + (timeout or self.args.startup_timeout)
        while not all(e.wait(0.1) for e in self._ready_events):
            dead = [p for p in self.procs if not p.is_alive()]
            if dead:
                self.last_error = (f"worker {dead[0].name} exited with code {dead[0].exitcode} during start-up"
                                   f"{self._oom_note(dead)} (phases: {self.startup.snapshot()})")
                self._kill_all()
                self.state = "failed"
                raise WorkerStartError(self.last_error)
            budgets = self.startup_budgets
            scale = float(getattr(self.args, "startup_phase_timeout_scale", 1.0) or 1.0)
            if scale != 1.0:                     # slow storage or a very large checkpoint: stretch every phase's limit
                from .startup_phases import DEFAULT_BUDGETS
                budgets = {k: v * scale for k, v in (budgets or DEFAULT_BUDGETS).items()}
            stalled = self.startup.stalled(budgets)
            if stalled:
                slot, phase, sec, limit = stalled[0]
                who = f"rank {slot}" if slot < self.args.world_size else "the server"
                self.last_error = (f"start-up stalled: {who} has been in phase '{phase}' for {sec:.0f} s "
                                   f"(budget {limit:.0f} s)")
                self._dump_stacks()
                self._kill_all()
                self.state = "failed"
                raise WorkerStartError(self.last_error)
            if time.monotonic() > deadline:
                self.last_error = "workers did not become ready before --startup-timeout"
                self._kill_all()
                self.state = "failed"
                raise WorkerStartError(self.last_error)
        self.state = "ready"
        self._monitor_stop.clear()
        self._monitor = threading.Thread(target=self._monitor_loop, name="worker-monitor", daemon=True)
        self._monitor.start()
        if self.args.watchdog_timeout > 0:
            self.watchdog = Watchdog(lambda: self.feed.value, self.args.watchdog_timeout, self._on_stall,
                                     armed=lambda: self.state == "ready" and bool(self._hooks.get("has_work", lambda: False)()))
            self.watchdog.start()

    def _create_host_region(self) -> None:
        """The node's host KV region belongs to the server: every worker of the cohort attaches to the same pages
        and the same prefix coordinator.  Created with the cohort for GPU deployments with a host tier
        (--host-kv-cache-size > 0) and dropped with it: pages that a dead worker's parked rows still reference
        cannot be told from live ones, so a restart starts from an empty region."""
        a = self.args
        if self.host_region is not None or a.host_kv_cache_size <= 0 or a.device == "cpu":
            return
        try:
            import torch
            if a.device == "auto" and not torch.cuda.is_available():
                return
            from ..config import get_model_config
            from ..core import native
            from ..runtime.kv_cache import host_page_bytes
            cfg = get_model_config(a.model) if isinstance(a.model, str) else a.model
            page_bytes = host_page_bytes(cfg, a.page_size)
            pages = int(a.host_kv_cache_size * (1 << 30)) // page_bytes
            if pages <= 0:
                return
            self.host_region = native.HostPagedKV(pages, page_bytes, 2 * pages)
            a.host_kv_region = f"/proc/{os.getpid()}/fd/{self.host_region.fd}"
            from ..utils import eventlog
            eventlog.get_log().info("server.host_kv_region", pages=pages, page_bytes=page_bytes, path=a.host_kv_region)
        except Exception as exc:                          # noqa: BLE001 - workers fall back to private regions
            self.host_region = None
            a.host_kv_region = ""
            from ..utils import eventlog
            eventlog.get_log().warning("server.host_kv_region_failed", error=str(exc))

    def _load_weight_store(self) -> None:
        """Checkpoint weights are read once per node, not once per worker: the server stages the converted
        checkpoint (optional copy to a local directory with a verified manifest), reads its shards with parallel
        readers into one shared region and hands workers the region's descriptor and tensor index; a worker's
        loader then returns views of that memory.  The region survives worker restarts.
        (batchgen/server/worker_manager.py: the server owns the weight memfd; server/weight_store_staging.py.)"""
        a = self.args
        if not a.converted_ckpt_dir or not a.shared_weight_store or self.weight_store is not None:
            return
        from ..core import native
        from ..utils import eventlog
        from . import weight_store_staging as staging
        log = eventlog.get_log()
        src = a.converted_ckpt_dir
        if a.weight_store_stage_dir:
            staged = staging.stage_store(src, a.weight_store_stage_dir)
            problem = staging.verify_store(staged.root)
            if problem is not None:
                raise WorkerStartError(f"staged weight store is not usable: {problem}")
            log.info("server.weight_store_staged", root=staged.root, reused=staged.reused, copied_bytes=staged.copied_bytes)
            src = staged.root
        t0 = time.monotonic()
        store = native.ParameterStore(nbytes=native.ParameterStore.bytes_needed(src), huge_pages=True)
        loaded = store.load_converted(src, threads=8)
        self.weight_store = store
        a.param_store_path = f"/proc/{os.getpid()}/fd/{store.fd}"
        self.weight_index = store.export_index()
        log.info("server.weight_store_loaded", bytes=loaded, tensors=len(self.weight_index),
                 seconds=round(time.monotonic() - t0, 2), path=a.param_store_path)

    def _oom_note(self, procs) -> str:
        """', killed by the kernel OOM killer' when the kernel log says so for one of ``procs``."""
        if not any(p.exitcode in (-9, 137) for p in procs):
            return ""
        from . import oom_attribution
        rec = oom_attribution.attribute([p.pid for p in procs if p.pid], self.kernel_log_path)
        return f": {rec.describe()}" if rec is not None else ""

    def _dump_stacks(self) -> None:
        """Ask every live worker for a Python stack dump (they register SIGUSR1 with ``faulthandler``; the dump goes
        to the worker's log directory or stderr) before the cohort is killed."""
        import signal
        for p in self.procs:
            if p.is_alive() and p.pid:
                try:
                    os.kill(p.pid, signal.SIGUSR1)
                except OSError:
                    pass
        time.sleep(0.3)

    def _on_stall(self, elapsed: float) -> None:
        self.last_error = f"watchdog: no engine step for {elapsed:.1f} s while work was pending"
        self._dump_stacks()
        self._fail_cohort(self.last_error)

    def _monitor_loop(self) -> None:
        while not self._monitor_stop.wait(0.2):
            if self.state != "ready":
                continue
            dead = [p for p in self.procs if not p.is_alive()]
            if dead:
                self._fail_cohort(f"worker {dead[0].name} exited with code {dead[0].exitcode}{self._oom_note(dead)}")
                return

    def _fail_cohort(self, reason: str) -> None:
        with self._lock:
            if self.state != "ready":
                return
            self.state = "failed"
            self.last_error = reason
        self._kill_all()
        self._hook("fail_in_flight", reason)

    def _kill_all(self) -> None:
        for p in self.procs:
            if p.is_alive():
                p.terminate()
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.kill()

    def stop(self, timeout: float = 20.0) -> None:
        with self._lock:
            if self.state == "stopped":
                return
            self._monitor_stop.set()
            if self.watchdog is not None:
                self.watchdog.stop()
                self.watchdog = None
            self._shutdown.set()
            try:
                self.send({"type": "shutdown"})
            except Exception:  # noqa: BLE001
                pass
        for p in self.procs:
            p.join(timeout=timeout)
        self._kill_all()
        self.procs = []
        if self.host_region is not None:
            self.host_region.close()
            self.host_region = None
            self.args.host_kv_region = ""
        self.state = "stopped"

    def restart_workers(self, reason: str = "requested") -> int:
        """Replace the cohort; returns the new generation."""
        self.phase = "P0"
        self._hook("quiesce")
        self.phase = "P1"
        self._hook("fail_in_flight", f"workers restarting: {reason}")
        self.stop()
        # messages addressed to the old cohort must not reach the new one
        self.request_queues = [self.ctx.Queue() for _ in range(self.dp)]
        self.request_queue = self.request_queues[0]
        self.response_queue = self.ctx.Queue()
        self._hook("rebind_queues", self.request_queue, self.response_queue)
        self.phase = "P2"
        self.start()
        self._hook("resume")
        self.phase = "idle"
        return self.generation

    # ------------------------------------------------------------------ status
    def status(self) -> WorkerStatus:
        return WorkerStatus(state=self.state, generation=self.generation, world_size=self.args.world_size,
                            pids=[p.pid for p in self.procs if p.pid], last_error=self.last_error,
                            capacity=self.capacity)
