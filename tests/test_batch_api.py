"""Offline batch API, tokenisers, event log."""
import json
import os

import pytest
import torch

from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.runtime import batch_api
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.tokenization import (ByteTokenizer, IdTokenizer, get_tokenizer, parse_tool_calls,
                                                split_reasoning)
from batchgen_b200.utils import eventlog


def _engine():
    cfg = get_model_config("tiny-deepseek-v3")
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1,
                        enable_prefix_cache=True)
    return cfg, Engine(build_model(cfg, seed=0), ecfg, num_gpu_pages=64)


def test_submit_batch_file_round_trip(tmp_path):
    cfg, eng = _engine()
    tok = ByteTokenizer(cfg.vocab_size)
    lines = [
        {"custom_id": "a", "method": "POST", "url": "/v1/chat/completions",
         "body": {"model": "tiny", "messages": [{"role": "user", "content": "hello world"}], "max_tokens": 5,
                  "ignore_eos": True}},
        {"custom_id": "b", "method": "POST", "url": "/v1/completions",
         "body": {"model": "tiny", "prompt": "once upon a time", "max_completion_tokens": 3, "max_tokens": 9,
                  "ignore_eos": True}},
        {"custom_id": "c", "method": "POST", "url": "/v1/completions", "body": {"prompt": "x", "max_tokens": -1}},
    ]
    inp, outp = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    inp.write_text("\n".join(json.dumps(l) for l in lines) + "\n")
    counts = batch_api.submit_batch_file(eng, str(inp), str(outp), tok, batch_api.BatchOptions(max_decoding_length=7))
    assert counts == {"total": 3, "completed": 2, "failed": 1}
    items = {json.loads(l)["custom_id"]: json.loads(l) for l in outp.read_text().splitlines()}
    a, b, c = items["a"], items["b"], items["c"]
    assert a["response"]["status_code"] == 200 and a["error"] is None
    body = a["response"]["body"]
    assert body["object"] == "chat.completion" and body["choices"][0]["message"]["role"] == "assistant"
    assert body["usage"]["completion_tokens"] == 5 and body["choices"][0]["finish_reason"] == "length"
    assert body["usage"]["total_tokens"] == body["usage"]["prompt_tokens"] + 5
    assert "cached_tokens" in body["usage"]["prompt_tokens_details"]
    assert b["response"]["body"]["usage"]["completion_tokens"] == 3          # max_completion_tokens wins
    assert b["response"]["body"]["object"] == "text_completion"
    assert c["response"] is None and c["error"]["code"] == "invalid_request"


@pytest.mark.parametrize("bad,msg", [
    ("not json", "not valid JSON"),
    (json.dumps({"custom_id": "", "body": {}}), "custom_id"),
    (json.dumps({"custom_id": "x", "url": "/v1/embeddings", "body": {}}), "url"),
    (json.dumps({"custom_id": "x", "url": "/v1/chat/completions", "body": {"prompt": "p"}}), "messages"),
    (json.dumps({"custom_id": "x", "method": "GET", "body": {}}), "POST"),
])
def test_batch_file_validation(bad, msg):
    with pytest.raises(batch_api.BatchFormatError, match=msg):
        batch_api.parse_batch_lines([bad])


def test_duplicate_custom_id_rejected():
    l = json.dumps({"custom_id": "x", "url": "/v1/completions", "body": {"prompt": "1"}})
    with pytest.raises(batch_api.BatchFormatError, match="duplicate"):
        batch_api.parse_batch_lines([l, l])


def test_tokenizers_and_parsers():
    t = IdTokenizer(100)
    assert t.encode("1 2 3") == [1, 2, 3] and t.decode([4, 5]) == "4 5"
    with pytest.raises(ValueError):
        t.encode("100")
    b = ByteTokenizer(1024)
    assert b.decode(b.encode("héllo")) == "héllo"
    assert isinstance(get_tokenizer("bytes", 1024), ByteTokenizer)
    ids = b.apply_chat_template([{"role": "user", "content": "hi"}])
    assert "<|user|>" in b.decode(ids) and b.decode(ids).endswith("<|assistant|>\n")
    assert split_reasoning("<think>plan</think>answer") == ("plan", "answer")
    assert split_reasoning("no thoughts") == (None, "no thoughts")
    calls, rest = parse_tool_calls('ok <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>')
    assert calls[0]["function"]["name"] == "f" and json.loads(calls[0]["function"]["arguments"]) == {"x": 1}
    assert rest == "ok"


def test_eventlog_schema_and_flight_recorder(tmp_path):
    log = eventlog.EventLog("worker0", str(tmp_path), flight_recorder=True)
    with eventlog.batch_context("batch_1"):
        log.info("prefill.wave", tokens=128, seqs=4)
    log.emit("debug", "hidden")            # below the level: dropped
    log.error("boom", why="x" * 2000)      # longer than a flight-recorder slot
    path, fpath = log.path, log.flight.path
    log.close()
    recs = [json.loads(l) for l in open(path)]
    assert [r["event"] for r in recs] == ["prefill.wave", "boom"]
    for r in recs:
        eventlog.validate_record(r)
    assert recs[0]["batch_id"] == "batch_1" and recs[0]["fields"]["tokens"] == 128 and recs[1]["batch_id"] is None
    ring = eventlog.FlightRecorder.read(fpath)
    assert ring and ring[0]["event"] == "prefill.wave"
    c = eventlog.StepCounters(None, period=1000)
    c.bump("decode_steps")
    c.bump("decode_steps", 2)
    assert c.c["decode_steps"] == 3 and not c.maybe_flush() and c.maybe_flush(force=True)


def test_workload_profiles_and_driver_roundtrip(tmp_path):
    """Synthetic workload files of the benchmark configurations run through the offline batch API."""
    import json
    import subprocess
    import sys
    sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent.parent))
    from benchmarks import workloads as wl
    p = wl.scaled(wl.PROFILES["long-grouped"], 1 / 2048)
    lines = list(wl.batch_lines(p, 1000, seed=1))
    assert len(lines) == p.requests and p.groups >= 1
    a, b = json.loads(lines[0])["body"]["prompt"], json.loads(lines[1])["body"]["prompt"]
    assert a[: len(a) - p.suffix_tokens] == b[: len(b) - p.suffix_tokens]        # members of a group share the prefix
    assert wl.summary(wl.PROFILES["mixed-1k"])["decode_tokens_total"] == 512 * 1024
    path = tmp_path / "tiny.jsonl"
    path.write_text("\n".join(wl.batch_lines(wl.PROFILES["tiny"], 1024)) + "\n")
    root = str(__import__("pathlib").Path(__file__).resolve().parent.parent)
    out = subprocess.run([sys.executable, "benchmarks/batch_driver.py", str(path), "--model", "tiny-deepseek-v3"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["prompt_tokens"] == 8 * 32 and res["decode_tokens"] == 8 * 16 and res["bct_s"] > 0
    assert res["stats"]["completed"] == 8
