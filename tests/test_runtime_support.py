"""Sampling residency, lifespan rings, restart coordinator, runtime locks."""
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
