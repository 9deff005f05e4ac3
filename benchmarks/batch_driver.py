"""Batch-completion-time driver: runs one workload file through the framework's public batch API and reports
the client-observed wall time from the first request issued to the last completion received, plus token
throughput.

  offline          in-process: ``runtime.batch_api.submit_batch_file`` on an ``Engine`` built from a model preset
  server           against a running server: upload the file, create the batch, poll, download the results
  concurrent-chat  against a running server: ``--concurrency`` clients, each walking through its share of the
                   workload as the turns of one session (``/v1/sessions`` + ``/v1/turns``), one turn at a time

Reference parity: benchmarks/decode_batch_driver.py (``batch-api`` and ``concurrent-chat`` modes), benchmarks/README.md:7-18.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_offline(path: str, model: str, device: str, pages: int) -> dict:
    import torch

    from batchgen_b200.config import EngineConfig, get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.runtime import batch_api
    from batchgen_b200.runtime.engine import Engine
    from batchgen_b200.runtime.tokenization import get_tokenizer
    cfg = get_model_config(model)
    dtype = "bf16" if device.startswith("cuda") else "fp32"
    eng = Engine(build_model(cfg, device, dtype, seed=0), EngineConfig(page_size=64 if device.startswith("cuda") else 16),
                 num_gpu_pages=pages)
    out = tempfile.NamedTemporaryFile("w", suffix=".jsonl", delete=False).name
    t0 = time.perf_counter()
    stats = batch_api.submit_batch_file(eng, path, out, get_tokenizer("ids", cfg.vocab_size))
    if device.startswith("cuda"):
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return {"mode": "offline", "model": model, "bct_s": dt, "stats": stats, "output_file": out}


def run_server(path: str, url: str, timeout_s: float) -> dict:
    from batchgen_b200.server.client import BatchGenHttpClient as BatchGenClient
    c = BatchGenClient(url)
    t0 = time.perf_counter()
    batch = c.submit_batch(path, endpoint="/v1/completions", timeout=timeout_s)
    dt = time.perf_counter() - t0
    res = c.results(batch) if batch.get("output_file_id") else []
    return {"mode": "server", "bct_s": dt, "status": batch.get("status"), "completed": len(res),
            "request_counts": batch.get("request_counts")}


def run_concurrent_chat(path: str, url: str, timeout_s: float, concurrency: int, client=None) -> dict:
    """Every client owns a session and sends its requests as successive turns; the wall time runs from the first turn
    issued to the last answer.  ``client``: an existing ``BatchGenHttpClient`` (tests)."""
    import threading

    from batchgen_b200.server.client import BatchGenHttpClient as BatchGenClient
    c = client or BatchGenClient(url, timeout_s=timeout_s)
    reqs = [json.loads(l)["body"] for l in open(path) if l.strip()]
    shares = [reqs[i::concurrency] for i in range(concurrency) if reqs[i::concurrency]]
    lat, errors, lock = [], [], threading.Lock()

    def worker(share):
        try:
            sid = c.create_session()["id"]
            for body in share:
                t = time.perf_counter()
                c.turn(sid, **{k: v for k, v in body.items() if k != "model"})
                with lock:
                    lat.append(time.perf_counter() - t)
            c.close_session(sid)
        except Exception as e:  # noqa: BLE001 - reported in the result line
            with lock:
                errors.append(f"{type(e).__name__}: {e}")

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, args=(sh,)) for sh in shares]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s)
    dt = time.perf_counter() - t0
    lat.sort()
    pick = (lambda q: lat[min(len(lat) - 1, int(q * len(lat)))]) if lat else (lambda q: 0.0)
    return {"mode": "concurrent-chat", "bct_s": dt, "clients": len(shares), "turns": len(lat), "errors": errors[:3],
            "turn_latency_s": {"p50": pick(0.5), "p95": pick(0.95), "max": lat[-1] if lat else 0.0}}


def tokens_in(path: str):
    prompt = decode = 0
    with open(path) as f:
        for line in f:
            if line.strip():
                b = json.loads(line)["body"]
                prompt += len(b["prompt"]) if isinstance(b.get("prompt"), list) else 0
                decode += int(b.get("max_tokens", 0))
    return prompt, decode


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="batch completion time of one workload file")
    ap.add_argument("workload")
    ap.add_argument("--mode", choices=["offline", "server", "concurrent-chat"], default="offline")
    ap.add_argument("--concurrency", type=int, default=8, help="clients of the concurrent-chat mode")
    ap.add_argument("--model", default="tiny-deepseek-v3")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--pages", type=int, default=512)
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--timeout", type=float, default=3600.0)
    a = ap.parse_args(argv)
    if a.mode == "offline":
        res = run_offline(a.workload, a.model, a.device, a.pages)
    elif a.mode == "server":
        res = run_server(a.workload, a.url, a.timeout)
    else:
        res = run_concurrent_chat(a.workload, a.url, a.timeout, a.concurrency)
    p, d = tokens_in(a.workload)
    res.update(prompt_tokens=p, decode_tokens=d, total_tokens_per_s=(p + d) / res["bct_s"])
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
