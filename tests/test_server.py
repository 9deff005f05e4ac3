"""HTTP server end to end with a CPU worker process, plus the control-plane units."""
import json
import os
import signal
import time

import pytest
from fastapi.testclient import TestClient

from batchgen_b200.server.http_server import create_app
from batchgen_b200.server.pools import HIGH, IntakeFull, IntakePool, IntakeRequest, SchedulingPool
from batchgen_b200.server.server_args import ServerArgs, ServerArgsError, prepare_server_args, validate_server_args
from batchgen_b200.server.storage import StorageManager, StorageOwnershipError
from batchgen_b200.server.io_struct import BatchObject


def _args(tmp_path, **kw):
    base = dict(model="tiny-deepseek-v3", device="cpu", tokenizer="bytes", page_size=16, num_gpu_pages=192,
                initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1,
                storage_path=str(tmp_path / "store"), startup_timeout=120.0, watchdog_timeout=0.0,
                enable_prefix_cache=True, max_model_len=512)
    base.update(kw)
    return validate_server_args(ServerArgs(**base))


def _lines(n, max_tokens=4):
    return [{"custom_id": f"r{i}", "method": "POST", "url": "/v1/chat/completions",
             "body": {"model": "tiny", "messages": [{"role": "user", "content": f"question number {i}"}],
                      "max_tokens": max_tokens, "ignore_eos": True}} for i in range(n)]


def _upload(c, lines):
    data = ("\n".join(json.dumps(l) for l in lines) + "\n").encode()
    r = c.post("/v1/files", files={"file": ("in.jsonl", data, "application/jsonl")}, data={"purpose": "batch"})
    assert r.status_code == 200, r.text
    return r.json()


def _wait(c, bid, timeout=120):
    t0 = time.time()
    while time.time() - t0 < timeout:
        b = c.get(f"/v1/batches/{bid}").json()
        if b["status"] in ("completed", "failed", "cancelled"):
            return b
        time.sleep(0.1)
    raise AssertionError(f"batch stuck: {b}")


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("srv")
    app = create_app(_args(tmp))
    with TestClient(app) as c:
        assert c.get("/health").status_code == 200, c.get("/health").text
        yield c, app


def test_batch_round_trip_and_api_surface(server):
    c, app = server
    assert c.get("/v1/models").json()["data"][0]["id"] == "tiny-deepseek-v3"
    assert c.get("/v1/models/other").status_code == 404
    f = _upload(c, _lines(6))
    assert c.get(f"/v1/files/{f['id']}").json()["bytes"] == f["bytes"]
    assert _upload(c, _lines(6))["id"] == f["id"]                       # sha256 de-duplication
    r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions",
                                    "max_decoding_length": 9})
    assert r.status_code == 200, r.text
    b = _wait(c, r.json()["id"])
    assert b["status"] == "completed" and b["request_counts"] == {"total": 6, "completed": 6, "failed": 0}
    out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
    assert sorted(o["custom_id"] for o in out) == [f"r{i}" for i in range(6)]
    for o in out:
        body = o["response"]["body"]
        assert o["response"]["status_code"] == 200 and body["usage"]["completion_tokens"] == 4
        assert body["choices"][0]["finish_reason"] == "length"
    assert any(x["id"] == b["id"] for x in c.get("/v1/batches").json()["data"])
    st = c.get("/v1/pool/status").json()
    assert st["serving"] and st["scheduling_slots_used"] == 0
    assert c.get("/v1/workers/status").json()["state"] == "ready"
    assert c.post("/v1/inference").status_code == 410
    assert c.get("/v1/batches/nope").status_code == 404 and c.get("/v1/files/nope/content").status_code == 404
    assert c.post("/v1/batches", json={"input_file_id": "file-missing"}).status_code == 404


def test_python_client_against_the_server(server, tmp_path):
    """The client's blocking and step-by-step paths (the FastAPI test client stands in for the HTTP session)."""
    from batchgen_b200.server.client import BatchGenHttpClient, LegacyInferenceDeprecated
    c, app = server
    cl = BatchGenHttpClient("", session=c)
    assert cl.health_check() and cl.list_models()[0]["id"] == "tiny-deepseek-v3"
    out_path = tmp_path / "out.jsonl"
    done = cl.submit_batch(_lines(3), output_file_path=str(out_path), max_decoding_length=8)
    assert done["status"] == "completed" and len(out_path.read_text().splitlines()) == 3
    assert len(cl.results(done)) == 3
    f = cl.upload_file(_lines(2))
    b = cl.create_batch(f["id"], endpoint="/v1/chat/completions", temperature=0.0)
    assert b["status"] in ("validating", "in_progress", "finalizing", "completed")
    assert cl.wait_for_batch(b["id"], poll_s=0.1, timeout_s=120)["status"] == "completed"
    pending = cl.submit_batch(_lines(1), wait=False)
    assert cl.wait_for_batch(pending["id"], poll_s=0.1, timeout_s=120)["request_counts"]["completed"] == 1
    assert "state" in cl.workers_status()
    with pytest.raises(LegacyInferenceDeprecated):
        cl.submit_inference("x")


def test_concurrent_chat_driver_walks_sessions_against_the_server(server, tmp_path):
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))
    import batch_driver
    from batchgen_b200.server.client import BatchGenHttpClient
    c, app = server
    path = tmp_path / "chat.jsonl"
    path.write_text("\n".join(json.dumps(l) for l in _lines(6, max_tokens=3)) + "\n")
    res = batch_driver.run_concurrent_chat(str(path), "", 120.0, 3, client=BatchGenHttpClient("", session=c))
    assert res["turns"] == 6 and res["clients"] == 3 and not res["errors"], res
    assert res["turn_latency_s"]["max"] >= res["turn_latency_s"]["p50"] > 0


def test_invalid_file_and_per_request_errors(server):
    c, _ = server
    r = c.post("/v1/files", files={"file": ("bad.jsonl", b"{not json\n", "application/jsonl")}, data={"purpose": "batch"})
    assert r.status_code == 400
    lines = _lines(2)
    lines[1]["body"]["max_tokens"] = 100000            # exceeds the context budget -> error item, batch completes
    f = _upload(c, lines)
    b = _wait(c, c.post("/v1/batches", json={"input_file_id": f["id"]}).json()["id"])
    assert b["status"] == "completed" and b["request_counts"] == {"total": 2, "completed": 1, "failed": 1}
    out = {json.loads(l)["custom_id"]: json.loads(l) for l in
           c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()}
    assert out["r1"]["error"] is not None and out["r0"]["error"] is None


def test_sessions_and_turns_reuse_context(server):
    c, _ = server
    s = c.post("/v1/sessions", json={}).json()
    t1 = c.post("/v1/turns", json={"session_id": s["id"], "prompt": "a" * 40, "max_tokens": 3, "ignore_eos": True}).json()
    t2 = c.post("/v1/turns", json={"session_id": s["id"], "prompt": "b" * 10, "max_tokens": 3, "ignore_eos": True}).json()
    assert t1["turn_index"] == 0 and t2["turn_index"] == 1
    assert t2["usage"]["prompt_tokens"] == 40 + 3 + 10
    assert t2["usage"]["prompt_tokens_details"]["cached_tokens"] >= 32      # prefix pages of turn 1 re-used
    assert c.get(f"/v1/sessions/{s['id']}").json()["turns"] == 2
    assert c.post(f"/v1/sessions/{s['id']}/close").json()["status"] == "closed"
    assert c.post("/v1/turns", json={"session_id": s["id"], "prompt": "x"}).status_code == 410


def test_cancel_batch(server):
    c, _ = server
    f = _upload(c, _lines(3, max_tokens=200))
    bid = c.post("/v1/batches", json={"input_file_id": f["id"]}).json()["id"]
    time.sleep(0.3)
    assert c.post(f"/v1/batches/{bid}/cancel").json()["status"] in ("cancelling", "cancelled", "completed")
    b = _wait(c, bid)
    assert b["status"] in ("cancelled", "completed")
    assert b["request_counts"]["completed"] + b["request_counts"]["failed"] == 3


def test_worker_restart_and_worker_loss_fail_fast(server):
    c, app = server
    gen0 = c.get("/v1/workers/status").json()["generation"]
    r = c.post("/v1/workers/restart")
    assert r.status_code == 200 and r.json()["generation"] == gen0 + 1
    f = _upload(c, _lines(2))
    assert _wait(c, c.post("/v1/batches", json={"input_file_id": f["id"]}).json()["id"])["status"] == "completed"
    # host-side failure: the worker process dies between steps; the monitor fails the cohort and the batch
    f = _upload(c, _lines(2, max_tokens=400))
    bid = c.post("/v1/batches", json={"input_file_id": f["id"]}).json()["id"]
    time.sleep(0.5)
    os.kill(app.state.worker.procs[0].pid, signal.SIGKILL)
    b = _wait(c, bid)
    assert b["status"] == "failed" and b["errors"]["data"][0]["code"] == "worker_failure"
    assert c.get("/health").status_code == 503
    assert c.post("/v1/batches", json={"input_file_id": f["id"]}).status_code == 503
    assert c.post("/v1/workers/restart").status_code == 200          # recovery: a new generation serves again
    assert c.get("/health").status_code == 200


# ---------------------------------------------------------------------- units
def test_intake_pool_all_or_nothing_and_priority():
    p = IntakePool(4)
    mk = lambda b, i, pr=0: IntakeRequest(b, f"r{i}", [1], {}, pr)
    p.submit_batch([mk("a", 0), mk("a", 1)])
    with pytest.raises(IntakeFull):
        p.submit_batch([mk("b", i) for i in range(3)])
    assert len(p) == 2
    p.submit_batch([mk("c", 0, HIGH)])
    assert [r.batch_id for r in p.drain(2)] == ["c", "a"]
    p.submit_batch([mk("d", 0)])
    assert p.cancel_batch("a") == 1 and [r.batch_id for r in p.drain(10)] == ["d"]


def test_scheduling_pool_slots_and_dedupe():
    sp = SchedulingPool(2)
    ip = IntakePool(10)
    ip.submit_batch([IntakeRequest("b", f"r{i}", [1], {}) for i in range(3)])
    sp.register_batch("b", 3)
    got = sp.select_from_intake(ip)
    assert len(got) == 2 and sp.free == 0 and len(ip) == 1
    assert sp.record_request_result("b", "r0", True) == (True, False)
    assert sp.record_request_result("b", "r0", True) == (False, False)     # replayed result: ignored
    assert sp.free == 1
    assert len(sp.select_from_intake(ip)) == 1
    sp.record_request_result("b", "r1", False)
    assert sp.record_request_result("b", "r2", True) == (True, True)
    t = sp.trackers["b"]
    assert (t.completed, t.failed) == (2, 1) and sp.free == 2


def test_storage_ownership_and_orphans(tmp_path):
    s = StorageManager(str(tmp_path))
    s.acquire_ownership()
    with pytest.raises(StorageOwnershipError):
        StorageManager(str(tmp_path)).acquire_ownership()
    b = BatchObject(status="in_progress", input_file_id="x")
    s.save_batch(b)
    s.append_output(b.id, {"custom_id": "r0"})
    s.release_ownership()
    s2 = StorageManager(str(tmp_path))
    s2.acquire_ownership()
    assert s2.fail_orphaned_batches() == [b.id]
    got = s2.get_batch(b.id)
    assert got.status == "failed" and got.errors.data[0].code == "server_restart"
    assert json.loads(s2.read_file(got.output_file_id).decode())["custom_id"] == "r0"
    s2.release_ownership()


def test_server_args_validation(tmp_path):
    a = prepare_server_args(["--model", "deepseek-r1", "--world-size", "8", "--host-kv-cache-size", "64",
                             "--no-enable-cuda-graph", "--enable-prefix-cache"])
    assert a.world_size == 8 and not a.enable_cuda_graph and a.enable_prefix_cache
    assert a.engine_config().attn_tp_size == 8
    for bad in (dict(world_size=3), dict(nnodes=2), dict(model="nope"), dict(kv_dtype="int4"),
                dict(ep_offloading_ratio=0.5), dict(extension_gpu_page_buffer=1, decision_frequency_pages=2)):
        with pytest.raises(ServerArgsError):
            validate_server_args(ServerArgs(**bad))


def test_server_loads_checkpoint_once_into_the_shared_store(tmp_path):
    """With a converted checkpoint the server stages it, reads it once into a node-shared region and the worker
    builds its model from views of that region: same completions as a worker that reads the files itself."""
    from batchgen_b200.ckpt.converter import convert_dir, save_model_checkpoint
    from batchgen_b200.config import get_model_config
    from batchgen_b200.models.weights import WeightSource
    cfg = get_model_config("tiny-deepseek-v3")
    save_model_checkpoint(cfg, WeightSource(seed=5), str(tmp_path / "hf"), shard_layers=2)
    convert_dir(str(tmp_path / "hf"), str(tmp_path / "conv"), workers=2)
    texts = []
    for shared in (True, False):
        kw = dict(converted_ckpt_dir=str(tmp_path / "conv"), shared_weight_store=shared)
        if shared:
            kw["weight_store_stage_dir"] = str(tmp_path / "stage")
        app = create_app(_args(tmp_path / f"s{int(shared)}", **kw))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            wm = app.state.worker
            assert (wm.weight_store is not None) == shared
            if shared:
                assert len(wm.weight_index) > 50 and os.path.exists(tmp_path / "stage" / "MANIFEST.json")
            f = _upload(c, _lines(3, max_tokens=6))
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"])
            assert b["status"] == "completed", b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            texts.append(sorted((o["custom_id"], o["response"]["body"]["choices"][0]["message"]["content"]) for o in out))
    assert texts[0] == texts[1]


def test_two_rank_cpu_cohort_reads_prompts_from_the_shared_token_book(tmp_path):
    """Two gloo ranks: rank 0 writes prompts into the node-shared token book, the follower reads them from there
    (the step broadcast carries offsets only); completions equal those of the one-rank server."""
    texts = []
    for world in (1, 2):
        app = create_app(_args(tmp_path / f"w{world}", world_size=world,
                               dist_init_addr=f"127.0.0.1:{29640 + world}", enable_prefix_cache=False))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            f = _upload(c, _lines(4, max_tokens=5))
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"])
            assert b["status"] == "completed" and b["request_counts"]["completed"] == 4, b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            texts.append(sorted((o["custom_id"], o["response"]["body"]["choices"][0]["message"]["content"]) for o in out))
    assert texts[0] == texts[1]


def test_data_parallel_cohorts_share_the_batch(tmp_path):
    """--dp-size 2 on two CPU ranks: two independent engines, requests spread by the sum of squared prompt lengths,
    a session's turns stay on one cohort, results equal those of the single-engine server."""
    texts = []
    for dp in (1, 2):
        app = create_app(_args(tmp_path / f"dp{dp}", world_size=dp, dp_size=dp, dist_init_addr=f"127.0.0.1:{29660 + 4 * dp}"))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            f = _upload(c, _lines(8, max_tokens=5))
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"])
            assert b["status"] == "completed" and b["request_counts"]["completed"] == 8, b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            texts.append(sorted((o["custom_id"], o["response"]["body"]["choices"][0]["message"]["content"]) for o in out))
            sched = app.state.scheduler
            if dp == 2:
                assert sched.dp_assigned[0] > 0 and sched.dp_assigned[1] > 0 and sum(sched.dp_assigned) == 8
                s = c.post("/v1/sessions", json={}).json()
                for turn in range(2):
                    t = c.post("/v1/turns", json={"session_id": s["id"], "prompt": "x" * 40, "max_tokens": 3,
                                                  "ignore_eos": True}).json()
                assert t["usage"]["prompt_tokens_details"]["cached_tokens"] >= 32     # same cohort: context reused
                assert len(sched._session_cohort) == 1
                assert all(v == 0 for v in sched._dp_load)                            # every completion came back
    assert texts[0] == texts[1]


def test_deepseek_v4_model_serves_chat_batches_in_its_own_format(tmp_path):
    """The server with a DeepSeek-V4 model on CPU workers: state slots for window / compressor state, prefix cache
    off, prompts rendered in the family's chat format (byte tokenizer), a batch completes; two ranks (attention
    replicated, experts expert-parallel over gloo) produce the tokens of one rank."""
    texts = []
    for world in (1, 2):
        app = create_app(_args(tmp_path / f"w{world}", model="tiny-deepseek-v4", enable_prefix_cache=False,
                               world_size=world, dist_init_addr=f"127.0.0.1:{29680 + world}"))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            f = _upload(c, _lines(5, max_tokens=6))
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"])
            assert b["status"] == "completed" and b["request_counts"]["completed"] == 5, b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            out.sort(key=lambda o: o["custom_id"])
            usage = out[0]["response"]["body"]["usage"]
            prompt = "<｜begin▁of▁sentence｜><｜User｜>question number 0<｜Assistant｜><think>"
            assert usage["prompt_tokens"] == len(prompt.encode("utf-8")) and usage["completion_tokens"] == 6
            texts.append([o["response"]["body"]["choices"][0]["message"]["content"] for o in out])
    assert texts[0] == texts[1]


def test_oversubscribed_device_pool_with_a_host_tier_completes_with_the_same_outputs(tmp_path):
    """Server-level oversubscription: a device pool that holds a fraction of the batch's KV plus a host tier; rows are
    parked, resumed and (when the host tier is full too) evicted and recomputed, and every request still returns the
    text of the unconstrained server."""
    texts, stats = [], []
    lines = [{"custom_id": f"r{i}", "method": "POST", "url": "/v1/chat/completions",
              "body": {"model": "tiny", "messages": [{"role": "user", "content": f"request {i}: " + "lorem ipsum " * (2 + i % 3)}],
                       "max_tokens": 40, "ignore_eos": True}} for i in range(10)]
    for name, kw in (("big", dict(num_gpu_pages=512)),
                     ("small", dict(num_gpu_pages=26, host_kv_cache_size=0.0002, max_decode_batch=8))):
        app = create_app(_args(tmp_path / name, enable_prefix_cache=False, **kw))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            f = _upload(c, lines)
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"], timeout=240)
            assert b["status"] == "completed" and b["request_counts"]["completed"] == 10, b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            texts.append(sorted((o["custom_id"], o["response"]["body"]["choices"][0]["message"]["content"]) for o in out))
            done = time.time()
            beat = None
            while time.time() - done < 15:                   # the worker's next heartbeat carries the engine counters
                beat = app.state.scheduler.last_heartbeat
                if beat and beat["ts"] >= done:
                    break
                time.sleep(0.2)
            stats.append(beat["stats"])
    assert texts[0] == texts[1]
    assert stats[0]["holds"] == 0 and stats[0]["evictions"] == 0
    assert stats[1]["holds"] + stats[1]["evictions"] > 0, stats[1]


def test_parked_rows_of_a_loaded_cohort_move_to_an_idle_cohort(tmp_path):
    """--dp-size 2: every request lands on cohort 0 (cohort 1 is made to look loaded), whose small device pool parks
    rows in its host tier; the heartbeats show parked rows on one side and an idle engine on the other, the server
    hands rows over (packed to files, adopted under new sequence numbers) and all outputs equal the one-engine run."""
    lines = [{"custom_id": f"r{i}", "method": "POST", "url": "/v1/chat/completions",
              "body": {"model": "tiny", "messages": [{"role": "user", "content": f"request {i}: " + "lorem ipsum " * (2 + i % 3)}],
                       "max_tokens": 100, "ignore_eos": True}} for i in range(8)]
    texts = []
    for dp in (1, 2):
        kw = dict(num_gpu_pages=512) if dp == 1 else dict(num_gpu_pages=20, host_kv_cache_size=0.0004, max_decode_batch=8,
                                                         heartbeat_interval=0.1)
        app = create_app(_args(tmp_path / f"dp{dp}", enable_prefix_cache=False, world_size=dp, dp_size=dp,
                               dist_init_addr=f"127.0.0.1:{29700 + 4 * dp}", **kw))
        with TestClient(app) as c:
            assert c.get("/health").status_code == 200, c.get("/health").text
            sched = app.state.scheduler
            if dp == 2:
                sched._dp_load[1] = 10 ** 15                      # cohort 1 looks loaded: the batch goes to cohort 0
            f = _upload(c, lines)
            r = c.post("/v1/batches", json={"input_file_id": f["id"], "endpoint": "/v1/chat/completions"})
            b = _wait(c, r.json()["id"], timeout=300)
            assert b["status"] == "completed" and b["request_counts"]["completed"] == 8, b
            out = [json.loads(l) for l in c.get(f"/v1/files/{b['output_file_id']}/content").text.splitlines()]
            texts.append(sorted((o["custom_id"], o["response"]["body"]["choices"][0]["message"]["content"]) for o in out))
            if dp == 2:
                assert sched.dp_assigned == [8, 0]
                assert sched.migrated_rows > 0, sched._cohort_stats
                assert not sched._handover
    assert texts[0] == texts[1]


def test_cohort_assignment_keeps_prefix_families_together_when_prefix_reuse_is_on():
    from types import SimpleNamespace
    from batchgen_b200.server.batch_scheduler import BatchScheduler
    sched = BatchScheduler.__new__(BatchScheduler)
    sched._dp_load = [0, 0]
    fam_a, fam_b = list(range(100, 180)), list(range(300, 380))
    prompts = [fam_a + [i] * 5 for i in range(4)] + [fam_b + [i] * 9 for i in range(4)] + [[7, 8, 9]]
    sched.args = SimpleNamespace(enable_prefix_cache=True, page_size=16)
    got = sched._assign_cohorts(prompts, 2)
    assert len(set(got[:4])) == 1 and len(set(got[4:8])) == 1 and got[0] != got[4]
    sched.args = SimpleNamespace(enable_prefix_cache=False, page_size=16)
    spread = sched._assign_cohorts(prompts, 2)
    assert len(set(spread[:4])) == 2                       # without reuse the family is spread by cost
    sched._dp_load = [10 ** 9, 0]
    sched.args = SimpleNamespace(enable_prefix_cache=True, page_size=16)
    assert set(sched._assign_cohorts(prompts, 2)) == {1}   # the loaded cohort gets nothing


def test_flags_of_the_reference_server_are_understood():
    from batchgen_b200.server.server_args import REFERENCE_ACCEPTED
    a = prepare_server_args(["--listen-ip", "0.0.0.0", "--listen-port", "9001", "--max-pool-size", "2048",
                             "--watchdog-heartbeat-interval", "2.5", "--runtime-mode", "exclusive",
                             "--input-ids-pool-size-gb", "0.5", "--enable-prepack", "--fast-init", "--gpu-arch", "sm_100a",
                             "--adaptive-chunk", "--adaptive-chunk-min", "512", "--adaptive-chunk-multiplier", "2.0",
                             "--startup-phase-timeout-scale", "3"])
    assert (a.host, a.port, a.max_intake_capacity, a.heartbeat_interval, a.query_book_mb) == ("0.0.0.0", 9001, 2048, 2.5, 512)
    assert a.accepted_reference_flags == ["enable_prepack", "fast_init", "gpu_arch"]
    assert all(k in REFERENCE_ACCEPTED for k in a.accepted_reference_flags)
    e = a.engine_config()
    assert e.adaptive_chunk and e.adaptive_chunk_min == 512 and e.adaptive_chunk_multiplier == 2.0
    assert a.startup_phase_timeout_scale == 3.0
    from batchgen_b200.models import build_model
    from batchgen_b200.config import get_model_config
    from batchgen_b200.runtime.engine import Engine
    eng = Engine(build_model(get_model_config("tiny-deepseek-v3"), seed=0), e, num_gpu_pages=32)
    assert eng.chunk_sizer.min_chunk == 512 and eng.chunk_sizer.multiplier == 2.0
