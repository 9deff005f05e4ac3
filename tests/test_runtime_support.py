"""Sampling residency, lifespan rings, restart coordinator, runtime locks."""
import os
import threading
import time

import pytest
import torch

from batchgen_b200.runtime.sampling_residency import (DecodeSamplingResidency, SamplingResidencyRowError,
                                                      SamplingResidencyShapeError)
from batchgen_b200.server import restart_coordinator as rc
from batchgen_b200.server import runtime_locks as rl
from batchgen_b200.utils.lifespan import LifespanRecorder, SeqEvent


def test_sampling_residency_uploads_only_on_change():
    res = DecodeSamplingResidency(8, "cpu", verify=True)
    rows = [0, 1, 2]
    params = [{"temperature": 0.0}, {"temperature": 0.7, "top_p": 0.9}, {"temperature": 1.0, "top_k": 40}]
    v = res.view(rows, params, 1, 1)
    assert v.temperature.tolist() == pytest.approx([0.0, 0.7, 1.0]) and v.top_k.tolist() == [0, 0, 40]
    assert not v.all_greedy and v.any_top_k and v.any_top_p
    res.view(rows, params, 1, 1)
    assert (res.uploads, res.hits) == (1, 1)
    rows2 = [2, 0]                                               # rebound list after a page boundary
    v = res.view(rows2, [params[2], params[0]], 1, 2)
    assert v.temperature.tolist() == pytest.approx([1.0, 0.0]) and res.uploads == 2
    assert res.view([5], [{"temperature": 0}], 2, 3).all_greedy
    with pytest.raises(SamplingResidencyShapeError):
        res.view([0, 1], [params[0]], 3, 3)
    with pytest.raises(SamplingResidencyRowError):
        res.view([0], [None], 4, 4)
    # same key, same list object, but different parameters: verify mode catches the stale cache
    same = [7]
    res.view(same, [{"temperature": 0.5}], 9, 9)
    with pytest.raises(SamplingResidencyRowError):
        res.view(same, [{"temperature": 0.9}], 9, 9)


def test_lifespan_ring_and_anomalies(tmp_path):
    off = LifespanRecorder(enabled=False)
    off.record("a", SeqEvent.CREATED)
    assert off.events("a") == []
    rec = LifespanRecorder(enabled=True, max_events=4, dump_dir=str(tmp_path))
    for e in (SeqEvent.CREATED, SeqEvent.PREFILL_START, SeqEvent.PREFILL_DONE, SeqEvent.DECODE_START, SeqEvent.KV_APPEND):
        rec.record("a", e, 1)
    assert [e for _, e, _, _ in rec.events("a")] == [SeqEvent.PREFILL_START, SeqEvent.PREFILL_DONE,
                                                     SeqEvent.DECODE_START, SeqEvent.KV_APPEND]
    assert rec.check_context("a", 10, 10)
    assert not rec.check_context("a", 10, 9) and (tmp_path / "lifespan_a.json").exists()
    assert rec.check_repetition("a", list(range(40)))
    assert not rec.check_repetition("a", [1, 2] + [5, 6] * 8)
    rec.forget("a")
    assert rec.events("a") == []


def test_restart_phases_across_nodes_and_failure_reporting():
    store = rc.InMemoryStore()
    nodes = [rc.RestartCoordinator(n, 3, store) for n in range(3)]
    order = []
    req = nodes[0].begin_restart(5.0)

    def follower(c):
        r = None
        while r is None:
            r = c.poll_request()
            time.sleep(0.005)
        c.run_phases(r, {"teardown": lambda: order.append(("teardown", c.node_rank))})

    ts = [threading.Thread(target=follower, args=(c,)) for c in nodes[1:]]
    [t.start() for t in ts]
    nodes[0].run_phases(req, {"teardown": lambda: order.append(("teardown", 0))})
    [t.join(10) for t in ts]
    assert sorted(order) == [("teardown", 0), ("teardown", 1), ("teardown", 2)] and all(c.epoch == 1 for c in nodes)
    # a failing node is named to the others instead of a silent timeout
    req = nodes[0].begin_restart(5.0)
    nodes[2].poll_request()
    nodes[2].fail_phase(req.epoch, "quiesce", "spawn failed")
    with pytest.raises(rc.PeerRestartError) as e:
        nodes[0].barrier(req.epoch, "quiesce", req.deadline)
    assert e.value.node == 2 and "spawn failed" in e.value.reason
    with pytest.raises(rc.RestartTimeout):
        nodes[0].barrier(req.epoch, "ready", time.monotonic() + 0.05)
    solo = rc.RestartCoordinator(0, 1)
    solo.run_phases(solo.begin_restart(1.0), {})
    assert solo.epoch == 1 and not solo.enabled


def test_liveness_by_incarnation_and_silence():
    store = rc.InMemoryStore()
    now = [0.0]
    a = rc.RestartCoordinator(0, 2, store, liveness_timeout_s=2.0, clock=lambda: now[0])
    b = rc.RestartCoordinator(1, 2, store, clock=lambda: now[0])
    b.beat()
    assert a.check_peers() is None
    now[0] = 1.5
    b.beat()
    assert a.check_peers() is None
    now[0] = 4.0                                                  # no beat for 2.5 s
    assert a.check_peers()[0] == 1 and "silent" in a.check_peers()[1]
    b.beat()
    assert a.check_peers() is None
    b2 = rc.RestartCoordinator(1, 2, store, clock=lambda: now[0])  # the process was replaced
    b2.beat()
    assert "replaced" in a.check_peers()[1]
    b2.publish_down(0, "worker crashed")
    assert "worker crashed" in a.check_peers()[1]


def test_runtime_locks_and_reclaim(tmp_path):
    root = tmp_path / "rt"
    run = root / "run-abc123"
    locks = rl.RuntimeLocks.acquire(root, run)
    with pytest.raises(rl.RuntimeLockError):
        rl.RuntimeLocks.acquire(root, run)                        # a second server in the same directory
    held = rl.hold_run_lock(run, create=True)
    assert not rl.run_is_dead(run)
    shm = tmp_path / "shm"
    shm.mkdir()
    (shm / "bg_run-abc123_kv").write_bytes(b"x")
    (shm / "other").write_bytes(b"y")
    assert rl.reclaim_dead_runs(root, [shm]) == []                # the run is alive
    rl.release_run_lock(held)
    locks.close()
    assert rl.run_is_dead(run)
    assert rl.reclaim_dead_runs(root, [shm]) == ["run-abc123"]
    assert not (shm / "bg_run-abc123_kv").exists() and (shm / "other").exists()
    with pytest.raises(rl.RuntimeLockError):
        rl.hold_run_lock(tmp_path / "nowhere")


def test_process_utils_and_hugepage_plan():
    import multiprocessing as mp
    import os
    import signal

    from batchgen_b200.server import process_utils as pu
    assert pu.hugepage_plan(3 << 30, free_1g=4).kind == "1g"
    assert pu.hugepage_plan(3 << 30, free_1g=2, free_2m=2000).kind == "2m"
    assert pu.hugepage_plan(3 << 30).kind == "base" and pu.hugepage_plan(100 << 20, free_1g=8, free_2m=100).kind == "2m"
    assert set(pu.read_hugepage_pools()) == {"free_2m", "free_1g"}
    ctx = mp.get_context("fork")
    q = ctx.Queue()

    def middle():
        def grandchild():
            pu.die_with_parent(signal.SIGKILL)
            q.put(os.getpid())
            import time
            time.sleep(60)
        p = ctx.Process(target=grandchild)
        p.start()
        q.put(("ready", None))
        import time
        time.sleep(60)

    m = ctx.Process(target=middle)
    m.start()
    got = [q.get(timeout=20), q.get(timeout=20)]
    gpid = next(g for g in got if isinstance(g, int))
    m.kill()                                                      # the server dies hard ...
    m.join(10)
    import time
    for _ in range(100):                                          # ... and its worker follows
        try:
            os.kill(gpid, 0)
            time.sleep(0.05)
        except ProcessLookupError:
            break
    else:
        os.kill(gpid, signal.SIGKILL)
        raise AssertionError("grandchild survived its parent")


def test_launch_readiness_gates(tmp_path):
    import socket

    from batchgen_b200.server import launch_readiness as lr
    rep = lr.check_node(None, str(tmp_path / "run"), str(tmp_path / "store"), "127.0.0.1", [], gpus=2, gpu_count_fn=lambda: 1)
    assert not rep.ok and [f.name for f in rep.failures()] == ["gpus"]
    assert not lr.gate_model_dir(str(tmp_path)).ok
    (tmp_path / "m.bin").write_bytes(b"x")
    (tmp_path / "m.json").write_text("{}")
    assert lr.gate_model_dir(str(tmp_path)).ok
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        s.listen(1)
        port = s.getsockname()[1]
        assert not lr.gate_port_free("127.0.0.1", port).ok
    t = [0.0]
    res = lr.gate_path_appears(str(tmp_path / "never"), 1.0, clock=lambda: t[0], sleep=lambda d: t.__setitem__(0, t[0] + d))
    assert not res.ok and "did not appear" in res.detail
    assert lr.gate_free_space("space", str(tmp_path), 1).ok and not lr.gate_free_space("space", str(tmp_path), 1 << 60).ok
    assert '"ok": false' in rep.to_json()


def test_weight_store_staging_is_idempotent_and_detects_damage(tmp_path):
    from batchgen_b200.server import weight_store_staging as ws
    src = tmp_path / "src"
    src.mkdir()
    for i in range(4):
        (src / f"shard{i}.bin").write_bytes(bytes([i]) * (1000 + i))
        (src / f"shard{i}.json").write_text(f'{{"i": {i}}}')
    dst = tmp_path / "tmpfs"
    a = ws.stage_store(str(src), str(dst))
    assert not a.reused and a.copied_bytes > 4000 and ws.verify_store(str(dst), check_digests=True) is None
    b = ws.stage_store(str(src), str(dst))
    assert b.reused and b.copied_bytes == 0 and b.listing_digest == a.listing_digest
    (dst / "shard2.bin").write_bytes(b"short")
    assert "shard2.bin" in ws.verify_store(str(dst))
    c = ws.stage_store(str(src), str(dst))
    assert not c.reused and c.copied_bytes == 1002 and ws.verify_store(str(dst), True) is None
    part = ws.stage_store(str(src), str(tmp_path / "node1"), partition=(1, 2))
    assert sorted(part.files) == ["shard1.bin", "shard1.json", "shard3.bin", "shard3.json"]
    (src / "orphan.bin").write_bytes(b"x")
    import pytest as _pt
    with _pt.raises(FileNotFoundError):
        ws.stage_store(str(src), str(dst))


# ---------------------------------------------------------------------------------------------- lane leases
def test_lane_lease_handover_and_conflicts(tmp_path, monkeypatch):
    from batchgen_b200.server import runtime_lease as rl
    root = tmp_path / "lanes"
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    want = rl.expected_for_server(["GPU-aaa", "GPU-bbb"], 8000, 29500, tmp_path / "store")
    res = rl.LaneReservation.reserve("prod-a", want, lock_root=root)
    # a second launcher cannot take an overlapping lane
    other = rl.expected_for_server(["GPU-bbb"], 8001, 29501, tmp_path / "store2")
    with pytest.raises(rl.LaneLeaseError, match="held by another run"):
        rl.LaneReservation.reserve("prod-b", other, lock_root=root)
    # the server adopts exactly what it is about to use
    with pytest.raises(rl.LaneLeaseError, match="another instance"):
        rl.LaneLease.adopt(res.manifest_fd, "prod-x", want, lock_root=root)
    with pytest.raises(rl.LaneLeaseError, match="does not cover"):
        rl.LaneLease.adopt(res.manifest_fd, "prod-a", want | {"port:9"}, lock_root=root)
    lease = rl.LaneLease.adopt(res.manifest_fd, "prod-a", want, lock_root=root)
    assert lease.held == len(want) == 5
    lease.release()                                      # closes the shared descriptions: the lane is free again
    res2 = rl.LaneReservation.reserve("prod-b", other, lock_root=root)
    res2.release()


def test_lane_lease_rejects_foreign_descriptors_and_unsafe_root(tmp_path):
    import json
    from batchgen_b200.server import runtime_lease as rl
    root = tmp_path / "lanes"
    want = rl.resource_names(["GPU-x"], [1234], [])
    res = rl.LaneReservation.reserve("inst", want, lock_root=root)
    # a manifest that points a resource at some other file
    stray = os.open(tmp_path / "stray", os.O_RDWR | os.O_CREAT, 0o600)
    fake = dict(res.fds)
    fake["port:1234"] = stray
    mfd = os.open(tmp_path / "m.json", os.O_RDWR | os.O_CREAT, 0o600)
    os.pwrite(mfd, json.dumps({"version": 1, "instance_id": "inst", "resources": fake}).encode(), 0)
    with pytest.raises(rl.LaneLeaseError, match="not its lock file"):
        rl.LaneLease.adopt(mfd, "inst", want, lock_root=root)
    os.chmod(root, 0o755)
    with pytest.raises(rl.LaneLeaseError, match="mode 0700"):
        rl.LaneLease.adopt(res.manifest_fd, "inst", want, lock_root=root)
    os.chmod(root, 0o700)
    res.release()
    os.close(stray)
    os.close(mfd)


def test_run_identity_names():
    from batchgen_b200.server import runtime_lease as rl
    a = rl.RunIdentity.create("prod-a")
    b = rl.RunIdentity.create("prod-a")
    assert a.run_id != b.run_id and a.shm_name("host_kv").startswith(f"bgb200_prod-a_{a.run_id}.")
    assert a.runtime_dir != b.runtime_dir
    for bad in ("", "Prod", "-x", "a" * 49):
        with pytest.raises(ValueError):
            rl.RunIdentity.create(bad)
    with pytest.raises(ValueError):
        rl.RunIdentity.create("ok", run_id="xyz")
    with pytest.raises(ValueError):
        rl.RunIdentity.create("ok", mode="both")


# ---------------------------------------------------------------------------------------------- run guard
def test_run_guard_locks_instance_adopts_lease_and_reclaims(tmp_path, monkeypatch):
    """The launcher path: one server per instance id, the lane lease checked against the server's own arguments,
    workers join the run, and the next start reclaims a run that nobody holds any more."""
    from batchgen_b200.server import run_guard, runtime_lease as rl, runtime_locks as locks
    from batchgen_b200.server.server_args import ServerArgs
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    root, lanes = tmp_path / "rt", tmp_path / "lanes"
    args = ServerArgs(instance_id="prod-a", runtime_root=str(root), port=8123, dist_init_addr="127.0.0.1:29611",
                      storage_path=str(tmp_path / "store"), lane_gpus="GPU-aaa,GPU-bbb", lane_lock_root=str(lanes))
    want = rl.expected_for_server(["GPU-aaa", "GPU-bbb"], 8123, 29611, tmp_path / "store")
    res = rl.LaneReservation.reserve("prod-a", want, lock_root=lanes)
    args.lane_manifest_fd = res.manifest_fd
    guard = run_guard.acquire(args)
    assert guard.lease is not None and guard.lease.held == 5
    assert args.runtime_dir == str(guard.run_dir) and args.run_id == guard.identity.run_id
    worker_lock = run_guard.join_run(args)                    # what every worker process does
    assert worker_lock is not None and not locks.run_is_dead(guard.run_dir)
    # a second server of the same instance is refused while the first one lives
    again = ServerArgs(instance_id="prod-a", runtime_root=str(root), port=8124)
    with pytest.raises(locks.RuntimeLockError):
        run_guard.acquire(again)
    # shared mode without a lease is refused
    shared = ServerArgs(instance_id="prod-b", runtime_root=str(root), port=8125, run_mode="shared")
    with pytest.raises(rl.LaneLeaseError):
        run_guard.acquire(shared)
    dead_run = guard.run_dir.name
    worker_lock.close()
    guard.close()
    nxt = run_guard.acquire(ServerArgs(instance_id="prod-a", runtime_root=str(root), port=8123))
    assert dead_run in nxt.reclaimed and nxt.lease is None
    assert run_guard.join_run(ServerArgs()) is None           # unguarded server (in-process tests)
    nxt.close()


# ---------------------------------------------------------------------------------------------- start-up phases, OOM, step ring
def test_startup_record_names_the_stalled_phase():
    from batchgen_b200.server import startup_phases as sp
    rec = sp.StartupRecord(3)
    assert rec.read(0) is None and rec.stalled() == []
    rec.enter(0, "communicator-init")
    rec.enter(1, "model-build")
    t = rec.read(1)[1]
    assert rec.read(0)[0] == "communicator-init" and rec.snapshot()[1][0] == "model-build"
    # rank 1 has sat in model-build past its budget; rank 0 moved on in time, slot 2 never started
    rec.enter(0, "serving")
    got = rec.stalled({"model-build": 5.0, "communicator-init": 5.0}, now=t + 9.0)
    assert [(s, p) for s, p, _, _ in got] == [(1, "model-build")] and 8.9 < got[0][2] < 9.5 and got[0][3] == 5.0
    assert rec.stalled({"model-build": 50.0}, now=t + 9.0) == []
    with rec.phase(2, "kv-pool"):
        assert rec.read(2)[0] == "kv-pool"
    null = sp.record_of(object())
    null.enter(0, "model-build")                           # a worker without a manager reports to nobody


def test_worker_manager_fails_a_start_that_sits_in_one_phase(tmp_path):
    """A worker that never leaves communicator-init: the manager names rank and phase instead of waiting for the
    total start-up timeout."""
    from batchgen_b200.server.server_args import ServerArgs
    from batchgen_b200.server.worker_manager import WorkerManager, WorkerStartError
    args = ServerArgs(model="tiny-deepseek-v3", device="cpu", startup_timeout=60.0, storage_path=str(tmp_path))
    wm = WorkerManager(args, worker_target=_stuck_worker)
    wm.startup_budgets = {"communicator-init": 1.0}
    t0 = time.monotonic()
    with pytest.raises(WorkerStartError, match="rank 0 has been in phase 'communicator-init'"):
        wm.start()
    assert time.monotonic() - t0 < 30 and wm.state == "failed"


def _stuck_worker(rank, world, args, rq, wq, ready, shutdown, feed):
    from batchgen_b200.server.startup_phases import record_of
    record_of(args).enter(rank, "communicator-init")
    time.sleep(120)


def test_oom_attribution_reads_the_kernel_log(tmp_path):
    from batchgen_b200.server import oom_attribution as oa
    log = tmp_path / "kmsg"
    log.write_text(
        "6,1200,5000,-;usb 1-1: new device\\n"
        "3,1201,6000,-;Out of memory: Killed process 4242 (bg-worker-1) total-vm:9000000kB, anon-rss:73400320kB, file-rss:0kB\\n"
        "6,1202,7000,-;oom-kill:constraint=CONSTRAINT_NONE,nodemask=(null),task=python,pid=777,uid=0\\n")
    rec = oa.attribute([1, 4242], str(log))
    assert rec is not None and rec.pid == 4242 and rec.comm == "bg-worker-1" and rec.anon_rss_kb == 73400320
    assert "OOM killer" in rec.describe() and "70.0 GiB" in rec.describe()
    assert oa.attribute([777], str(log)).comm == "python"
    assert oa.attribute([5], str(log)) is None and oa.attribute([5], str(tmp_path / "missing")) is None


def test_step_ring_keeps_the_latest_events():
    from batchgen_b200.utils.step_ring import StepRing
    r = StepRing(4)
    for i in range(6):
        r.record("decode" if i % 2 else "prefill", rows=i, tokens=10 * i, seconds=0.001 * (i + 1))
    assert len(r) == 4 and [e["rows"] for e in r.tail(10)] == [2, 3, 4, 5]
    s = r.summary()
    assert s["decode"]["events"] == 2 and s["decode"]["tokens"] == 80 and abs(s["decode"]["max_ms"] - 6.0) < 1e-6


def test_model_contract_names_every_violated_kernel_rule():
    from batchgen_b200.config import get_model_config
    from batchgen_b200.server.preflight import PreflightError, model_contract
    notes = model_contract(get_model_config("deepseek-v3-671b"), 8, True, "fused")
    assert any("split-KV" in n for n in notes) and any("fused NVLink path" in n for n in notes)
    assert any("persistent" in n for n in model_contract(get_model_config("deepseek-v3-671b"), 2, True))
    assert any("NCCL layout" in n for n in model_contract(get_model_config("glm-5.3-fp8"), 8, True, "fused"))
    model_contract(get_model_config("tiny-minimax"), 1, True)
    with pytest.raises(PreflightError) as e:                       # the CPU-sized test preset has no kernel geometry
        model_contract(get_model_config("tiny-deepseek-v3"), 1, True)
    assert "kv_lora_rank 512" in str(e.value) and "heads per rank" in str(e.value)
    assert model_contract(get_model_config("tiny-deepseek-v3"), 1, False)      # fine on the reference path
    with pytest.raises(PreflightError, match="do not divide"):
        model_contract(get_model_config("minimax-m2.5"), 5, False)


def test_capture_window_brackets_the_requested_steps_once():
    from batchgen_b200.utils.capture_window import CaptureWindow, MemoryHistory, parse_window
    assert parse_window("3:5") == (3, 5) and parse_window("4:4") == (4, 4)
    assert parse_window("") is None and parse_window("5:3") is None and parse_window("x:1") is None and parse_window("7") is None
    events = []
    w = CaptureWindow((2, 4), start=lambda: events.append(("start", w.step)), stop=lambda: events.append(("stop", w.step)))
    for _ in range(8):
        w.before_step()
        w.after_step()
    assert events == [("start", 2), ("stop", 4)] and w.done and not w.active
    off = CaptureWindow(None, start=lambda: events.append("x"), stop=lambda: events.append("y"))
    for _ in range(3):
        off.before_step(); off.after_step()
    assert len(events) == 2
    assert MemoryHistory("").dump("t") is None              # off: nothing is written


def test_plan_cohort_handover_picks_the_loaded_and_the_idle_cohort():
    from batchgen_b200.runtime.scheduler import plan_cohort_handover as plan
    assert plan({}) is None
    assert plan({0: {"parked": 0, "live": 5, "host_free": 9}, 1: {"parked": 0, "live": 0, "host_free": 9}}) is None
    assert plan({0: {"parked": 4, "live": 9, "host_free": 1}, 1: {"parked": 0, "live": 2, "host_free": 9}}) is None   # nobody idle
    assert plan({0: {"parked": 5, "live": 9, "host_free": 1}, 1: {"parked": 0, "live": 0, "host_free": 9}}) == (0, 1, 2)
    assert plan({0: {"parked": 1, "live": 9, "host_free": 1}, 1: {"parked": 0, "live": 0, "host_free": 0},
                 2: {"parked": 0, "live": 0, "host_free": 7}}) == (0, 2, 1)
    assert plan({0: {"parked": 5, "live": 9, "host_free": 1}, 1: {"parked": 0, "live": 0, "host_free": 9}}, in_flight=[1]) is None


def test_parked_row_moves_between_two_engines_and_keeps_its_tokens():
    import torch
    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.runtime import kv_migration as mig
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.sequence import SamplingParams
    cfg = get_model_config("tiny-deepseek-v3")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(2, cfg.vocab_size, (32,), generator=g).tolist() for _ in range(6)]
    params = SamplingParams(max_new_tokens=48, ignore_eos=True)

    def mk(pages, host):
        ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1,
                            max_decode_batch=8)
        return Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=pages, num_host_pages=host)

    want = mk(256, 0).generate(prompts, params)
    a, b = mk(14, 64), mk(64, 64)
    outs = {}
    a.on_complete = b.on_complete = lambda s: outs.__setitem__(tuple(s.prompt_ids), list(s.output_ids))
    for p in prompts:
        a.add_request(p, params)
    moved = 0
    for _ in range(4000):
        if a.has_work():
            a.step()
        if b.has_work():
            b.step()
        rows = mig.parked_rows(a)
        if rows and moved < 3:
            before = a.host_kv.alloc.num_free
            payload = mig.export_sequence(a, rows[0])
            assert a.host_kv.alloc.num_free == before + payload["header"]["n_pages"]
            s = mig.import_sequence(b, payload)
            assert s.status.name == "ON_HOLD" and s.global_idx in b.seqs
            moved += 1
        if not a.has_work() and not b.has_work():
            break
    assert moved > 0
    assert [outs[tuple(p)] for p in prompts] == want
    assert a.kv.alloc.num_used == 0 and b.kv.alloc.num_used == 0


def test_deployment_plan_preflight_reports_and_refuses(monkeypatch):
    import torch
    from batchgen_b200.server import preflight
    from batchgen_b200.server.server_args import ServerArgs
    assert "CPU run" in preflight.deployment_plan(ServerArgs(model="tiny-deepseek-v3", device="cpu"))[0]
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(preflight, "_gpu_name", lambda: "NVIDIA B200")
    line = preflight.deployment_plan(ServerArgs(model="deepseek-v3-671b", device="cuda", world_size=8))[0]
    assert "b200, 8 GPUs per cohort" in line and "experts 76.1 GiB" in line
    with pytest.raises(preflight.PreflightError) as e:
        preflight.deployment_plan(ServerArgs(model="kimi-k3", device="cuda", world_size=8))
    assert "ep-offloading-ratio" in str(e.value)
    ok = preflight.deployment_plan(ServerArgs(model="kimi-k3", device="cuda", world_size=8, num_gpu_pages=1024))[0]
    assert "continuing" in ok
    two = preflight.deployment_plan(ServerArgs(model="gpt-oss-120b", device="cuda", world_size=8, dp_size=2))[0]
    assert "4 GPUs per cohort" in two


def test_bench_reference_arm_prints_one_json_line_and_exits_zero():
    """The reference arm either runs the installed reference or says in one line why it cannot; it never fails."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stderr[-500:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and ("unavailable" in line or "value" in line)


def test_rows_of_tiers_that_cannot_be_packed_are_never_offered_for_hand_over():
    import torch
    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.runtime import kv_migration as mig
    from batchgen_b200.runtime.engine import Engine
    ecfg = EngineConfig(page_size=16, max_decode_batch=4, max_state_slots=4)
    v4 = Engine(build_model(get_model_config("tiny-deepseek-v4"), seed=0), ecfg, num_gpu_pages=16, num_host_pages=16)
    assert not mig.can_export(v4) and mig.parked_rows(v4) == []
    plain = Engine(build_model(get_model_config("tiny-deepseek-v3"), seed=0), EngineConfig(page_size=16), num_gpu_pages=16)
    assert not mig.can_export(plain) and mig.parked_rows(plain) == []      # no host tier at all
