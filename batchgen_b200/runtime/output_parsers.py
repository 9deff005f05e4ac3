"""Tool-call markup of the model families' completions -> OpenAI ``tool_calls``.

Each family writes function calls in its own markup (the chat templates teach it in the prompt); the batch API returns
them in one shape.  ``parse_tool_calls(text, fmt)`` returns (calls, text without the call markup):

* ``json``      ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Qwen / Hermes style, the default)
* ``glm``       ``<tool_call>name<arg_key>k</arg_key><arg_value>v</arg_value>...</tool_call>``; values that parse as
                JSON are taken as JSON, the rest as strings
* ``kimi``      ``<|tool_calls_section_begin|><|tool_call_begin|>functions.name:0<|tool_call_argument_begin|>{json}
                <|tool_call_end|>...<|tool_calls_section_end|>``; the call id is the model's own (``functions.name:0``)
* ``minimax``   ``<minimax:tool_call><invoke name="f"><parameter name="k">v</parameter></invoke></minimax:tool_call>``
* ``deepseek``  ``<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>name<｜tool▁sep｜>{json}<｜tool▁call▁end｜>...``, also the
                older form ``function<｜tool▁sep｜>name`` followed by a fenced ``json`` block

Reference parity: the per-family ``parse_tool_calls`` of batchgen/models/glm/glm5/tokenizer.py:170-203,
moonshotai/kimi_k25/tokenizer.py:236-284, minimax/minimax_m25/tokenizer.py:107-152, deepseek/deepseekv3/tokenizer.py:113-141
and the default in batchgen/config/base_tokenizer.py.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Tuple

FAMILY_FORMAT = {"glm5": "glm", "kimi_k3": "kimi", "kimi_k25": "kimi", "minimax": "minimax", "deepseek_v3": "deepseek",
                 "deepseek_v2": "deepseek"}

_JSON_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_GLM_CALL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)
_GLM_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)
_KIMI_SECTION = re.compile(r"<\|tool_calls_section_begin\|>(.*?)<\|tool_calls_section_end\|>", re.S)
_KIMI_CALL = re.compile(r"<\|tool_call_begin\|>\s*([\w\.\-]+:\d+)\s*<\|tool_call_argument_begin\|>\s*(.*?)\s*<\|tool_call_end\|>", re.S)
_MM_BLOCK = re.compile(r"<minimax:tool_call>(.*?)</minimax:tool_call>", re.S)
_MM_INVOKE = re.compile(r'<invoke\s+name="([^"]+)">(.*?)</invoke>', re.S)
_MM_PARAM = re.compile(r'<parameter\s+name="([^"]+)">(.*?)</parameter>', re.S)
_DS_SECTION = re.compile(r"<｜tool▁calls▁begin｜>(.*?)(?:<｜tool▁calls▁end｜>|$)", re.S)
_DS_CALL = re.compile(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁call▁end｜>", re.S)
_FENCE = re.compile(r"```(?:json)?\s*(.*?)\s*```", re.S)


def _value(raw: str) -> Any:
    raw = raw.strip()
    try:
        return json.loads(raw)
    except ValueError:
        return raw


def _call(n: int, name: str, arguments: Any, call_id: str = "") -> Dict:
    args = arguments if isinstance(arguments, str) else json.dumps(arguments, ensure_ascii=False)
    return {"id": call_id or f"call_{n}", "type": "function", "function": {"name": name, "arguments": args}}


def parse_tool_calls(text: str, fmt: str = "json") -> Tuple[List[Dict], str]:
    calls: List[Dict] = []
    if fmt == "glm":
        for m in _GLM_CALL.finditer(text):
            raw = m.group(1).strip()
            k = raw.find("<arg_key>")
            name = (raw if k < 0 else raw[:k]).strip()
            if name.startswith("{"):                      # a JSON call inside the same tags
                try:
                    obj = json.loads(raw)
                    calls.append(_call(len(calls), obj.get("name", ""), obj.get("arguments", {})))
                    continue
                except ValueError:
                    pass
            args = {a.group(1).strip(): _value(a.group(2)) for a in _GLM_ARG.finditer(raw)}
            calls.append(_call(len(calls), name, args))
        return calls, _GLM_CALL.sub("", text).strip()
    if fmt == "kimi":
        for sec in _KIMI_SECTION.finditer(text):
            for m in _KIMI_CALL.finditer(sec.group(1)):
                call_id, raw = m.group(1), m.group(2)
                name = call_id.rsplit(":", 1)[0]
                name = name.split(".", 1)[1] if name.startswith("functions.") else name
                calls.append(_call(len(calls), name, raw, call_id))
        return calls, _KIMI_SECTION.sub("", text).strip()
    if fmt == "minimax":
        for block in _MM_BLOCK.finditer(text):
            for inv in _MM_INVOKE.finditer(block.group(1)):
                args = {p.group(1): _value(p.group(2)) for p in _MM_PARAM.finditer(inv.group(2))}
                calls.append(_call(len(calls), inv.group(1), args))
        return calls, _MM_BLOCK.sub("", text).strip()
    if fmt == "deepseek":
        for sec in _DS_SECTION.finditer(text):
            for m in _DS_CALL.finditer(sec.group(1)):
                head, _, rest = m.group(1).partition("<｜tool▁sep｜>")
                if head.strip() == "function":            # function<sep>name \n ```json {...} ```
                    name, _, tail = rest.partition("\n")
                    fence = _FENCE.search(tail)
                    raw = fence.group(1) if fence else tail.strip()
                else:
                    name, raw = head, rest.strip()
                calls.append(_call(len(calls), name.strip(), raw))
        return calls, _DS_SECTION.sub("", text).strip()
    for m in _JSON_CALL.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except ValueError:
            continue
        calls.append(_call(len(calls), obj.get("name", ""), obj.get("arguments", {})))
    return calls, _JSON_CALL.sub("", text).strip()


def audit_output_file(path: str, fmt: str = "json") -> Dict[str, int]:
    """Re-parse the raw texts of a batch output file (written without ``--parse-tool-call``) and count what the parser
    finds: items, items with calls, calls, calls whose arguments are not valid JSON, and items that still contain an
    opening call marker after parsing (markup the parser did not understand)."""
    markers = {"json": "<tool_call>", "glm": "<tool_call>", "kimi": "<|tool_call_begin|>", "minimax": "<minimax:tool_call>",
               "deepseek": "<｜tool▁call▁begin｜>"}
    out = {"items": 0, "with_calls": 0, "calls": 0, "bad_arguments": 0, "leftover_markup": 0}
    with open(path, encoding="utf-8") as f:
        for line in f:
            if not line.strip():
                continue
            item = json.loads(line)
            body = ((item.get("response") or {}).get("body") or {})
            for choice in body.get("choices", []):
                text = (choice.get("message") or {}).get("content") or choice.get("text") or ""
                calls, rest = parse_tool_calls(text, fmt)
                out["items"] += 1
                out["with_calls"] += bool(calls)
                out["calls"] += len(calls)
                for c in calls:
                    try:
                        json.loads(c["function"]["arguments"])
                    except ValueError:
                        out["bad_arguments"] += 1
                out["leftover_markup"] += markers.get(fmt, "<tool_call>") in rest
    return out


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="count the tool calls a batch output file's texts parse into")
    ap.add_argument("output_file")
    ap.add_argument("--format", default="json", choices=["json", "glm", "kimi", "minimax", "deepseek"])
    a = ap.parse_args()
    print(json.dumps(audit_output_file(a.output_file, a.format)))
