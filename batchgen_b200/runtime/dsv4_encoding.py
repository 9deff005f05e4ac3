"""Prompt encoding of the DeepSeek-V4 chat format and the parser of its completions.

The format is plain text around a few special tokens:

    <BOS>{system}[tools block]<｜latest_reminder｜>{reminder}<｜User｜>{user}<｜Assistant｜>{think}{answer}[tool calls]<EOS>...

* ``thinking`` mode opens the assistant turn with ``<think>`` and closes the reasoning with ``</think>``; ``chat`` mode
  (and assistant turns whose reasoning is dropped) put ``</think>`` right after ``<｜Assistant｜>``.
* Reasoning of assistant turns before the last user turn is dropped unless tools are declared (tool conversations
  need the whole chain).
* Tools are declared on a ``system`` or ``developer`` message (``tools`` field, OpenAI format) and rendered as a schema
  block after that message's text; a ``developer`` message is a user turn.
* Tool calls are written in DSML markup: one ``invoke`` per call, one ``parameter`` per argument; strings are written
  raw (``string="true"``), everything else as JSON (``string="false"``).  Tool results come back inside the next user
  turn as ``<tool_result>`` blocks, in the order of the calls they answer.
* A ``task`` field adds a quick-instruction token: ``action`` goes after the assistant prefix, ``title`` after an
  assistant turn's EOS, the others right after the user text.
* ``reasoning_effort="max"`` puts a fixed instruction paragraph before the system text.

Reference parity: batchgen/models/deepseek/deepseekv4_flash/tokenizer.py (chat rendering for the DeepSeek-V4 family) and
the format description it ships (assets/encoding/README.md); checked against that directory's golden prompt files.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Optional, Tuple

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
USER = "<｜User｜>"
ASSISTANT = "<｜Assistant｜>"
REMINDER = "<｜latest_reminder｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
TASK_TOKENS = {"action": "<｜action｜>", "title": "<｜title｜>", "query": "<｜query｜>", "authority": "<｜authority｜>",
               "domain": "<｜domain｜>", "extracted_url": "<｜extracted_url｜>", "read_url": "<｜read_url｜>"}

MAX_EFFORT_PREFIX = (
    "Reasoning Effort: Absolute maximum with no shortcuts permitted.\n"
    "You MUST be very thorough in your thinking and comprehensively decompose the problem to resolve the root cause, "
    "rigorously stress-testing your logic against all potential paths, edge cases, and adversarial scenarios.\n"
    "Explicitly write out your entire deliberation process, documenting every intermediate step, considered "
    "alternative, and rejected hypothesis to ensure absolutely no assumption is left unchecked.\n")

_TOOLS_HEAD = f"""## Tools

You have access to a set of tools to help answer the user's question. You can invoke tools by writing a "<{DSML}tool_calls>" block like the following:

<{DSML}tool_calls>
<{DSML}invoke name="$TOOL_NAME">
<{DSML}parameter name="$PARAMETER_NAME" string="true|false">$PARAMETER_VALUE</{DSML}parameter>
...
</{DSML}invoke>
<{DSML}invoke name="$TOOL_NAME2">
...
</{DSML}invoke>
</{DSML}tool_calls>

String parameters should be specified as is and set `string="true"`. For all other types (numbers, booleans, arrays, objects), pass the value in JSON format and set `string="false"`.

If thinking_mode is enabled (triggered by <think>), you MUST output your complete reasoning inside <think>...</think> BEFORE any tool calls or final response.

Otherwise, output directly after </think> with tool calls or final response.

### Available Tool Schemas

"""
_TOOLS_TAIL = "\n\nYou MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n"


def _dumps(value: Any) -> str:
    return json.dumps(value, ensure_ascii=False)


def render_tools(tools: List[Dict]) -> str:
    """The schema block appended to the message that declares ``tools`` (one JSON line per function)."""
    lines = [_dumps(t["function"] if "function" in t else t) for t in tools]
    return "\n\n" + _TOOLS_HEAD + "\n".join(lines) + _TOOLS_TAIL


def render_tool_calls(tool_calls: List[Dict]) -> str:
    out = [f"<{DSML}tool_calls>\n"]
    for call in tool_calls:
        fn = call.get("function", call)
        args = fn.get("arguments", {})
        if isinstance(args, str):
            args = json.loads(args) if args.strip() else {}
        out.append(f'<{DSML}invoke name="{fn["name"]}">\n')
        for key, value in args.items():
            if isinstance(value, str):
                out.append(f'<{DSML}parameter name="{key}" string="true">{value}</{DSML}parameter>\n')
            else:
                out.append(f'<{DSML}parameter name="{key}" string="false">{_dumps(value)}</{DSML}parameter>\n')
        out.append(f"</{DSML}invoke>\n")
    out.append(f"</{DSML}tool_calls>")
    return "".join(out)


def _text(content: Any) -> str:
    if isinstance(content, list):                   # OpenAI content parts: keep the text ones
        return "".join(p.get("text", "") for p in content if isinstance(p, dict))
    return content or ""


def _ordered_tool_results(messages: List[Dict], start: int) -> Tuple[List[str], int]:
    """The run of ``tool`` messages that starts at ``start``, ordered like the calls of the assistant turn before
    it (results that carry no known call id keep their position)."""
    end = start
    while end < len(messages) and messages[end].get("role") == "tool":
        end += 1
    run = messages[start:end]
    order: Dict[str, int] = {}
    if start > 0 and messages[start - 1].get("role") == "assistant":
        for i, call in enumerate(messages[start - 1].get("tool_calls") or []):
            if call.get("id") is not None:
                order[call["id"]] = i
    keyed = sorted(range(len(run)), key=lambda i: (order.get(run[i].get("tool_call_id"), len(order) + i), i))
    return [_text(run[i].get("content")) for i in keyed], end


def encode_messages(messages: List[Dict], thinking_mode: str = "thinking", drop_thinking: bool = True,
                    reasoning_effort: Optional[str] = None, add_bos: bool = True) -> str:
    """Render a conversation.  When it ends with a user, developer or tool message the assistant prefix of the turn to
    generate is appended (``<think>`` in thinking mode, ``</think>`` in chat mode)."""
    if thinking_mode not in ("thinking", "chat"):
        raise ValueError("thinking_mode is 'thinking' or 'chat'")
    has_tools = any(m.get("tools") for m in messages if m.get("role") in ("system", "developer"))
    keep_all_reasoning = has_tools or not drop_thinking
    last_user = max((i for i, m in enumerate(messages) if m.get("role") in ("user", "developer")), default=-1)
    out: List[str] = [BOS] if add_bos else []
    if reasoning_effort == "max":
        out.append(MAX_EFFORT_PREFIX)
    pending_action = False          # the previous user turn asked for the action token
    after_title = False             # the previous assistant turn ended with the title token
    i = 0
    while i < len(messages):
        m = messages[i]
        role = m.get("role", "user")
        if role == "system":
            out.append(_text(m.get("content")))
            if m.get("tools"):
                out.append(render_tools(m["tools"]))
        elif role == "latest_reminder":
            out.append(REMINDER + _text(m.get("content")))
        elif role in ("user", "developer"):
            out.append(USER + _text(m.get("content")))
            if m.get("tools"):
                out.append(render_tools(m["tools"]))
            task = m.get("task")
            pending_action = task == "action"
            if task and task not in ("action", "title"):
                out.append(TASK_TOKENS[task])
        elif role == "tool":
            results, i = _ordered_tool_results(messages, i)
            out.append(USER + "\n\n".join(f"<tool_result>{r}</tool_result>" for r in results))
            pending_action = False
            continue
        elif role == "assistant":
            body = _text(m.get("content"))
            if m.get("tool_calls"):
                body += "\n\n" + render_tool_calls(m["tool_calls"])
            if after_title:                         # the generated title: no turn prefix
                out.append(body + EOS)
                after_title = False
            else:
                reasoning = m.get("reasoning_content")
                keep = thinking_mode == "thinking" and reasoning is not None and (keep_all_reasoning or i > last_user)
                think = THINK_OPEN + reasoning + THINK_CLOSE if keep else THINK_CLOSE
                out.append(ASSISTANT + think + (TASK_TOKENS["action"] if pending_action else "") + body + EOS)
            if m.get("task") == "title":
                out.append(TASK_TOKENS["title"])
                after_title = True
            pending_action = False
        else:
            raise ValueError(f"unknown role {role!r}")
        i += 1
    if messages and messages[-1].get("role") in ("user", "developer", "tool"):
        task = messages[-1].get("task")
        if not task or task == "action":
            out.append(ASSISTANT + (THINK_OPEN if thinking_mode == "thinking" else THINK_CLOSE))
            if task == "action":
                out.append(TASK_TOKENS["action"])
    return "".join(out)


_INVOKE = re.compile(rf'<{DSML}invoke name="([^"]*)">\n?(.*?)</{DSML}invoke>', re.S)
_PARAM = re.compile(rf'<{DSML}parameter name="([^"]*)" string="(true|false)">(.*?)</{DSML}parameter>', re.S)


def parse_completion(text: str, thinking_mode: str = "thinking") -> Dict[str, Any]:
    """Split a well-formed completion into reasoning, content and tool calls (OpenAI format, JSON-string arguments).
    In thinking mode the completion starts inside the reasoning block (the prompt ended with ``<think>``)."""
    if text.endswith(EOS):
        text = text[: -len(EOS)]
    reasoning = ""
    if thinking_mode == "thinking":
        if text.startswith(THINK_OPEN):
            text = text[len(THINK_OPEN):]
        if THINK_CLOSE in text:
            reasoning, text = text.split(THINK_CLOSE, 1)
    elif text.startswith(THINK_CLOSE):
        text = text[len(THINK_CLOSE):]
    calls: List[Dict] = []
    start = text.find(f"<{DSML}tool_calls>")
    if start >= 0:
        block = text[start:]
        text = text[:start]
        if text.endswith("\n\n"):
            text = text[:-2]
        for n, inv in enumerate(_INVOKE.finditer(block)):
            args = {}
            for key, is_str, raw in _PARAM.findall(inv.group(2)):
                args[key] = raw if is_str == "true" else json.loads(raw)
            calls.append({"id": f"call_{n}", "type": "function",
                          "function": {"name": inv.group(1), "arguments": _dumps(args)}})
    return {"role": "assistant", "reasoning_content": reasoning, "content": text, "tool_calls": calls}
