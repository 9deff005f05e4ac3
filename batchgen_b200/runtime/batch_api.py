"""Offline batch API: OpenAI-style batch JSONL in, results JSONL out.

Input line:  ``{"custom_id", "method": "POST", "url": "/v1/chat/completions" | "/v1/completions",
"body": {"model", "messages" | "prompt", "max_completion_tokens" | "max_tokens", "temperature", "top_p",
"top_k", "ignore_eos", ...}}``.  Length limit priority: per-request ``max_completion_tokens`` >
``max_tokens`` > the batch's ``max_decoding_length``.

Output line: ``{"id", "custom_id", "response": {"status_code", "body": {"id", "object", "model", "choices":
[{"index", "message" | "text", "finish_reason"}], "usage": {"prompt_tokens", "completion_tokens",
"total_tokens", "prompt_tokens_details": {"cached_tokens"}}}}, "error"}`` in completion order; a request
that fails validation yields an ``error`` item in the same file.

Reference parity: docs/input-format.md, docs/output-format.md, docs/batch-api.md:162-247; parsing and
validation batchgen/server/batch_scheduler.py:118-240, result items :2035-2184.
"""
from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

from .sequence import SamplingParams, Sequence
from .tokenization import parse_tool_calls, split_reasoning

ENDPOINTS = ("/v1/chat/completions", "/v1/completions")


class BatchFormatError(ValueError):
    pass


@dataclass
class BatchRequest:
    custom_id: str
    url: str
    body: Dict[str, Any]
    line_no: int = 0


@dataclass
class BatchOptions:
    endpoint: str = "/v1/chat/completions"
    max_decoding_length: int = 256
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    parse_thinking: bool = False
    parse_tool_call: bool = False
    include_special_tokens: bool = False
    model: str = ""
    tool_call_format: str = "json"              # json | glm | kimi | minimax | deepseek (runtime.output_parsers)


def parse_batch_lines(lines: Iterable[str], endpoint: Optional[str] = None) -> List[BatchRequest]:
    """Validate a batch file.  Raises ``BatchFormatError`` naming the first bad line."""
    out: List[BatchRequest] = []
    seen = set()
    for i, raw in enumerate(lines, 1):
        raw = raw.strip()
        if not raw:
            continue
        try:
            obj = json.loads(raw)
        except ValueError as e:
            raise BatchFormatError(f"line {i}: not valid JSON ({e})")
        if not isinstance(obj, dict):
            raise BatchFormatError(f"line {i}: expected an object")
        cid = obj.get("custom_id")
        if not isinstance(cid, str) or not cid:
            raise BatchFormatError(f"line {i}: custom_id must be a non-empty string")
        if cid in seen:
            raise BatchFormatError(f"line {i}: duplicate custom_id {cid!r}")
        seen.add(cid)
        if obj.get("method", "POST") != "POST":
            raise BatchFormatError(f"line {i}: method must be POST")
        url = obj.get("url", endpoint or ENDPOINTS[0])
        if url not in ENDPOINTS:
            raise BatchFormatError(f"line {i}: url must be one of {ENDPOINTS}")
        if endpoint and url != endpoint:
            raise BatchFormatError(f"line {i}: url {url} differs from the batch endpoint {endpoint}")
        body = obj.get("body")
        if not isinstance(body, dict):
            raise BatchFormatError(f"line {i}: body must be an object")
        if url == "/v1/chat/completions" and not isinstance(body.get("messages"), list):
            raise BatchFormatError(f"line {i}: chat requests need body.messages")
        if url == "/v1/completions" and "prompt" not in body:
            raise BatchFormatError(f"line {i}: completion requests need body.prompt")
        out.append(BatchRequest(cid, url, body, i))
    if not out:
        raise BatchFormatError("the batch file contains no requests")
    return out


def sampling_from_body(body: Dict[str, Any], opts: BatchOptions) -> SamplingParams:
    def pick(key, batch_default, fallback):
        v = body.get(key)
        if v is None:
            v = batch_default
        return fallback if v is None else v

    max_new = body.get("max_completion_tokens") or body.get("max_tokens") or opts.max_decoding_length
    if not isinstance(max_new, int) or max_new <= 0:
        raise BatchFormatError("max tokens must be a positive integer")
    temperature = float(pick("temperature", opts.temperature, 0.0))
    top_p = float(pick("top_p", opts.top_p, 1.0))
    top_k = int(pick("top_k", opts.top_k, 0))
    if temperature < 0 or not 0 < top_p <= 1 or top_k < 0:
        raise BatchFormatError("sampling parameters out of range")
    return SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, max_new_tokens=max_new,
                          ignore_eos=bool(body.get("ignore_eos", False)), seed=body.get("seed"))


def prompt_ids(req: BatchRequest, tokenizer) -> List[int]:
    if req.url == "/v1/chat/completions":
        kw = {}
        for k in ("enable_thinking", "reasoning_effort", "tools"):
            if k in req.body:
                kw[k] = req.body[k]
        try:
            return list(tokenizer.apply_chat_template(req.body["messages"], add_generation_prompt=True, **kw))
        except TypeError:
            return list(tokenizer.apply_chat_template(req.body["messages"], add_generation_prompt=True))
    p = req.body["prompt"]
    if isinstance(p, list) and p and all(isinstance(t, int) for t in p):
        return list(p)                      # pre-tokenised prompt (array of token ids), as the completions API allows
    return list(tokenizer.encode(p))


def result_item(seq: Sequence, req: BatchRequest, tokenizer, opts: BatchOptions) -> Dict[str, Any]:
    text = tokenizer.decode(seq.output_ids, skip_special_tokens=not opts.include_special_tokens)
    rid = "batch_req_" + uuid.uuid4().hex[:24]
    usage = {"prompt_tokens": len(seq.prompt_ids), "completion_tokens": len(seq.output_ids),
             "total_tokens": len(seq.prompt_ids) + len(seq.output_ids),
             "prompt_tokens_details": {"cached_tokens": seq.cached_prefix_tokens}}
    if req.url == "/v1/chat/completions":
        reasoning, content, tool_calls = None, text, None
        if hasattr(tokenizer, "parse_completion") and (opts.parse_thinking or opts.parse_tool_call):
            # the family's own completion format (DeepSeek-V4: reasoning up to </think>, DSML tool calls)
            parsed = tokenizer.parse_completion(text, enable_thinking=bool(req.body.get("enable_thinking", True)))
            reasoning = (parsed["reasoning_content"] or None) if opts.parse_thinking else None
            content = parsed["content"] if opts.parse_thinking else text
            tool_calls = parsed["tool_calls"] if opts.parse_tool_call else None
        elif opts.parse_thinking:
            reasoning, content = split_reasoning(text)
        if opts.parse_tool_call and not hasattr(tokenizer, "parse_completion"):
            from .output_parsers import parse_tool_calls as parse_family_calls
            tool_calls, content = parse_family_calls(content, opts.tool_call_format or "json")
        msg = {"role": "assistant", "content": content, "reasoning_content": reasoning,
               "tool_calls": tool_calls or None}
        choice = {"index": 0, "message": msg, "logprobs": None, "finish_reason": seq.finish_reason}
        obj = "chat.completion"
    else:
        choice = {"index": 0, "text": text, "logprobs": None, "finish_reason": seq.finish_reason}
        obj = "text_completion"
    body = {"id": "cmpl-" + uuid.uuid4().hex[:24], "object": obj, "created": int(time.time()),
            "model": req.body.get("model", opts.model), "choices": [choice], "usage": usage}
    return {"id": rid, "custom_id": req.custom_id, "response": {"status_code": 200, "request_id": rid, "body": body},
            "error": None}


def error_item(req: BatchRequest, message: str, code: str = "invalid_request") -> Dict[str, Any]:
    return {"id": "batch_req_" + uuid.uuid4().hex[:24], "custom_id": req.custom_id, "response": None,
            "error": {"code": code, "message": message}}


def run_batch(engine, requests: List[BatchRequest], tokenizer, opts: Optional[BatchOptions] = None,
              on_item: Optional[Callable[[Dict[str, Any]], None]] = None, batch_id: str = "") -> List[Dict[str, Any]]:
    """Run a parsed batch to completion on ``engine``.  Items are delivered to ``on_item`` (and collected)
    in completion order."""
    opts = opts or BatchOptions()
    items: List[Dict[str, Any]] = []
    by_idx: Dict[int, BatchRequest] = {}

    def deliver(item):
        items.append(item)
        if on_item is not None:
            on_item(item)

    prev_cb = engine.on_complete

    def completed(seq: Sequence):
        req = by_idx.get(seq.global_idx)
        if req is not None:
            if seq.finish_reason and seq.finish_reason.startswith("error"):
                deliver(error_item(req, seq.finish_reason, "engine_error"))
            else:
                deliver(result_item(seq, req, tokenizer, opts))
        if prev_cb is not None:
            prev_cb(seq)

    engine.on_complete = completed
    try:
        for req in requests:
            try:
                ids = prompt_ids(req, tokenizer)
                params = sampling_from_body(req.body, opts)
                seq = engine.add_request(ids, params, custom_id=req.custom_id, batch_id=batch_id)
                by_idx[seq.global_idx] = req
            except (ValueError, KeyError, TypeError) as e:
                deliver(error_item(req, str(e)))
        engine.run_to_completion()
    finally:
        engine.on_complete = prev_cb
    return items


def submit_batch_file(engine, input_path: str, output_path: str, tokenizer, opts: Optional[BatchOptions] = None) -> Dict[str, int]:
    """File-to-file offline batch: the call a user of the library makes.  The output is appended and
    flushed item by item, so a crash keeps everything completed so far."""
    import os
    opts = opts or BatchOptions()
    with open(input_path) as f:
        reqs = parse_batch_lines(f, None)
    counts = {"total": len(reqs), "completed": 0, "failed": 0}
    with open(output_path, "a") as out:
        def write(item):
            out.write(json.dumps(item) + "\n")
            out.flush()
            os.fsync(out.fileno())
            counts["failed" if item["error"] else "completed"] += 1
        run_batch(engine, reqs, tokenizer, opts, on_item=write)
    return counts
