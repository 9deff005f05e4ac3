"""The GPT-OSS "harmony" chat format: prompt rendering (messages, tools, tool-call history) and completion parsing.

A harmony prompt is a run of messages ``<|start|>{header}<|message|>{body}{terminator}``.  The header is a role, an
optional ``to={recipient}``, and for assistant / tool messages ``<|channel|>{analysis|commentary|final}`` (plus
``<|constrain|>json`` on tool calls); the terminator is ``<|end|>``, ``<|call|>`` after a tool call, or ``<|return|>``
at the end of a sampled final answer.

* The system text gets the line that names the valid channels; when tools are declared it also says that calls to
  ``functions`` go to the commentary channel, and a developer message follows with the tools written as
  TypeScript-like declarations inside ``namespace functions``.
* An assistant turn with tool calls renders as: reasoning on the analysis channel (only while its turn is still open:
  reasoning of turns that already ended in a final answer is dropped), an optional commentary preamble, one call
  message per call; a ``tool`` message renders as a message *from* ``functions.{name}`` *to* the assistant.
* JSON-schema parameters map to declarations: ``string`` / ``number`` (also for ``integer``) / ``boolean``, string
  enums as unions of literals, ``T[]``, nested objects, optional properties with ``?``, lists of scalar types as
  unions; ``title`` / ``description`` / string ``examples`` become comments and ``default`` a trailing comment.
  A schema outside that subset is declared ``any`` with the raw JSON schema in a comment, never a misleading type.

Reference parity: batchgen/models/openai/gpt_oss_120b/tokenizer.py (render_harmony_prompt, parse_harmony, thinking /
tool-call parsing) and harmony_tools.py (functions namespace); the expected texts of its unit tests are the checks.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

START, END, MESSAGE, CHANNEL, CONSTRAIN, CALL, RETURN = ("<|start|>", "<|end|>", "<|message|>", "<|channel|>",
                                                         "<|constrain|>", "<|call|>", "<|return|>")
SYSTEM_SUFFIX = "\n\n# Valid channels: analysis, commentary, final. Channel must be included for every message."
TOOL_NOTE = "\nCalls to these tools must go to the commentary channel: 'functions'."
NAMESPACE = "functions"

_SCALARS = {"string": "string", "number": "number", "integer": "number", "boolean": "boolean"}
_IGNORED = {"format", "minimum", "maximum", "exclusiveMinimum", "exclusiveMaximum", "multipleOf", "minLength",
            "maxLength", "pattern", "minItems", "maxItems", "uniqueItems", "minProperties", "maxProperties"}
_KNOWN = {"type", "enum", "items", "properties", "required", "additionalProperties", "description", "title", "examples",
          "default"} | _IGNORED


# ------------------------------------------------------------------------------------------ tools -> declarations
def _json(value: Any) -> str:
    """Compact JSON with floats written the short way (1e20, not 1e+20)."""
    if isinstance(value, bool) or value is None or isinstance(value, (int, str)):
        return json.dumps(value, ensure_ascii=False)
    if isinstance(value, float):
        return repr(value).replace("e+", "e")
    if isinstance(value, (list, tuple)):
        return "[" + ",".join(_json(v) for v in value) + "]"
    if isinstance(value, dict):
        return "{" + ",".join(json.dumps(str(k), ensure_ascii=False) + ":" + _json(v) for k, v in value.items()) + "}"
    return json.dumps(value, ensure_ascii=False)


def _comment(indent: str, text: str) -> str:
    return "".join(f"{indent}// {line}\n" for line in text.split("\n"))


def _supported(schema: Any) -> bool:
    if not isinstance(schema, dict) or any(k not in _KNOWN for k in schema):
        return False
    for k in ("title", "description"):
        if k in schema and not isinstance(schema[k], str):
            return False
    if "additionalProperties" in schema and not isinstance(schema["additionalProperties"], bool):
        return False
    t = schema.get("type")
    if t is None:
        return not any(k in schema for k in ("enum", "items", "properties"))
    if isinstance(t, list):
        return (bool(t) and all(x in _SCALARS or x == "null" for x in t) and any(x in _SCALARS for x in t)
                and "enum" not in schema)
    if t in _SCALARS:
        if "enum" in schema:
            e = schema["enum"]
            return t == "string" and isinstance(e, list) and bool(e) and all(isinstance(x, str) for x in e)
        return True
    if t == "array":
        items = schema.get("items")
        return items is None or (isinstance(items, dict) and _supported(items))
    if t == "object":
        props = schema.get("properties", {})
        return isinstance(props, dict)
    return False


def _type_expr(schema: Mapping, indent: str) -> str:
    """Declaration of a supported schema; ``indent`` is the indentation of the members of an object at this level."""
    t = schema.get("type")
    if t is None:
        return "any"
    if isinstance(t, list):
        return " | ".join(_SCALARS.get(x, "null") for x in t)
    if t in _SCALARS:
        if "enum" in schema:
            return " | ".join(f'"{v}"' for v in schema["enum"])
        return _SCALARS[t]
    if t == "array":
        items = schema.get("items")
        return "Array<any>" if items is None else _type_expr(items, indent) + "[]"
    head = (indent + "// " + schema["description"].replace("\n", "\n" + indent + "// ") + "\n") if "description" in schema else ""
    required = set(schema.get("required", []) or [])
    body = "".join(_property(k, v, k in required, indent) for k, v in schema.get("properties", {}).items())
    return f"{head}{{\n{body}{indent}}}"


def _property(key: str, schema: Any, required: bool, indent: str) -> str:
    out = ""
    if isinstance(schema, dict):
        if isinstance(schema.get("title"), str):
            out += _comment(indent, schema["title"]) + f"{indent}//\n"
        if isinstance(schema.get("description"), str):
            out += _comment(indent, schema["description"])
        examples = [e for e in schema.get("examples", []) or [] if isinstance(e, str)] if isinstance(schema.get("examples"), list) else []
        if examples:
            out += f"{indent}// Examples:\n" + "".join(f"{indent}// - {json.dumps(e, ensure_ascii=False)}\n" for e in examples)
    opt = "" if required else "?"
    if not _supported(schema):
        return out + f"{indent}// JSON schema: {json.dumps(schema, ensure_ascii=False)}\n{indent}{key}{opt}: any,\n"
    expr = _type_expr(schema, indent + "    ")
    line = f"{indent}{key}{opt}: {expr},"
    if "default" in schema:
        d = schema["default"]
        line += " // default: " + (d if ("enum" in schema and isinstance(d, str)) else _json(d))
    return out + line + "\n"


def validate_function_name(name: Any, where: str) -> str:
    if not isinstance(name, str) or not name:
        raise ValueError(f"{where}: function name must be a non-empty string")
    if re.search(r"\s", name):
        raise ValueError(f"{where}: function name {name!r} contains whitespace")
    return name


def render_functions_namespace(tools: Sequence[Any]) -> str:
    """OpenAI ``tools`` -> the developer message's ``# Tools`` section."""
    if not isinstance(tools, (list, tuple)):
        raise ValueError(f"tools must be a list, got {type(tools).__name__}")
    decls, seen = [], set()
    for i, tool in enumerate(tools):
        where = f"tools[{i}]"
        if not isinstance(tool, dict) or tool.get("type") != "function":
            raise ValueError(f'{where}: only {{"type": "function", ...}} tools are supported')
        fn = tool.get("function")
        if not isinstance(fn, dict):
            raise ValueError(f"{where}: 'function' must be an object")
        name = validate_function_name(fn.get("name"), where)
        if name in seen:
            raise ValueError(f"{where}: duplicate function name {name!r}")
        seen.add(name)
        desc = fn.get("description", "")
        if desc is None:
            desc = ""
        if not isinstance(desc, str):
            raise ValueError(f"{where}: description must be a string")
        text = _comment("", desc) if desc else ""
        if fn.get("parameters") is None:
            text += f"type {name} = () => any;"
        else:
            params = fn["parameters"]
            if not isinstance(params, dict):
                raise ValueError(f"{where}: parameters must be a JSON-schema object")
            if _supported(params):
                text += f"type {name} = (_: {_type_expr(params, '')}) => any;"
            else:
                text += f"// JSON schema: {json.dumps(params, ensure_ascii=False)}\ntype {name} = (_: any) => any;"
        decls.append(text)
    return "# Tools\n\n## functions\n\nnamespace functions {\n\n" + "\n\n".join(decls) + "\n\n} // namespace functions"


# ------------------------------------------------------------------------------------------ prompt rendering
def _msg(header: str, channel: Optional[str], body: str, terminator: str = END) -> str:
    return f"{START}{header}{'' if channel is None else CHANNEL + channel}{MESSAGE}{body}{terminator}"


def _text(message: dict, field: str, index: int, optional: bool = False) -> str:
    v = message.get(field)
    if v is None and optional:
        return ""
    if not isinstance(v, str):
        raise ValueError(f"messages[{index}]: {field!r} must be a string")
    return v


def _call_parts(call: Any, where: str) -> Tuple[str, str, Optional[str]]:
    if not isinstance(call, dict):
        raise ValueError(f"{where}: a tool call must be an object")
    if call.get("type", "function") != "function":
        raise ValueError(f"{where}: only function tool calls are supported")
    fn = call.get("function")
    if not isinstance(fn, dict):
        raise ValueError(f"{where}: 'function' must be an object")
    name = validate_function_name(fn.get("name"), where)
    args = fn.get("arguments")
    if not isinstance(args, str):
        raise ValueError(f"{where}: function.arguments must be the JSON-encoded string of the arguments")
    return name, args, call.get("id")


def render_harmony_prompt(messages: List[dict], tools: Optional[List[dict]] = None,
                          add_generation_prompt: bool = False) -> str:
    if not isinstance(messages, list):
        raise ValueError(f"messages must be a list, got {type(messages).__name__}")
    if tools is not None and not isinstance(tools, list):
        raise ValueError(f"tools must be a list, got {type(tools).__name__}")
    developer = _msg("developer", None, render_functions_namespace(tools)) if tools else None

    def has_calls(m) -> bool:
        return isinstance(m, dict) and m.get("role") == "assistant" and bool(m.get("tool_calls"))

    last_final = max((i for i, m in enumerate(messages)
                      if isinstance(m, dict) and m.get("role") == "assistant" and not has_calls(m)), default=-1)
    leading_system = bool(messages) and isinstance(messages[0], dict) and messages[0].get("role") == "system"
    parts: List[str] = [developer] if (developer is not None and not leading_system) else []
    names: Dict[str, str] = {}
    for i, m in enumerate(messages):
        if not isinstance(m, dict):
            raise ValueError(f"messages[{i}] must be an object, got {type(m).__name__}")
        role = m.get("role")
        if role == "system":
            body = _text(m, "content", i) + SYSTEM_SUFFIX
            first_with_tools = developer is not None and i == 0
            parts.append(_msg("system", None, body + (TOOL_NOTE if first_with_tools else "")))
            if first_with_tools:
                parts.append(developer)
        elif role == "user":
            parts.append(_msg("user", None, _text(m, "content", i)))
        elif role == "assistant" and not has_calls(m):
            parts.append(_msg("assistant", "final", _text(m, "content", i)))
        elif role == "assistant":
            calls = m["tool_calls"]
            if not isinstance(calls, list):
                raise ValueError(f"messages[{i}]: tool_calls must be a list")
            reasoning = _text(m, "reasoning_content", i, optional=True)
            if reasoning and i > last_final:
                parts.append(_msg("assistant", "analysis", reasoning))
            preamble = _text(m, "content", i, optional=True)
            if preamble:
                parts.append(_msg("assistant", "commentary", preamble))
            for j, call in enumerate(calls):
                name, args, cid = _call_parts(call, f"messages[{i}].tool_calls[{j}]")
                if cid is not None:
                    names[cid] = name
                parts.append(_msg(f"assistant to={NAMESPACE}.{name}", f"commentary {CONSTRAIN}json", args, CALL))
        elif role == "tool":
            where = f"messages[{i}] (tool)"
            cid, name = m.get("tool_call_id"), m.get("name")
            if cid is not None:
                if cid not in names:
                    raise ValueError(f"{where}: tool_call_id {cid!r} matches no earlier assistant tool call")
                if name is not None and name != names[cid]:
                    raise ValueError(f"{where}: name {name!r} disagrees with tool_call_id {cid!r}, which called {names[cid]!r}")
                name = names[cid]
            elif name is None:
                raise ValueError(f"{where}: needs tool_call_id (or name) to say which function returned this result")
            else:
                name = validate_function_name(name, where)
            parts.append(_msg(f"{NAMESPACE}.{name} to=assistant", "commentary", _text(m, "content", i)))
        else:
            raise ValueError(f"messages[{i}]: role {role!r} is not supported by the GPT-OSS chat format "
                             f"(system, user, assistant, tool)")
    if add_generation_prompt:
        parts.append(START + "assistant")
    return "".join(parts)


# ------------------------------------------------------------------------------------------ parsing
@dataclass
class HarmonyMessage:
    role: str = "assistant"
    channel: Optional[str] = None
    recipient: Optional[str] = None
    content_type: Optional[str] = None
    body: str = ""
    terminator: Optional[str] = None      # None: the text ended inside this message
    header_complete: bool = True          # False: the text ended before <|message|>

    @property
    def kind(self) -> str:
        if self.recipient and self.recipient.startswith(NAMESPACE + "."):
            return "tool_call"
        if self.channel == "analysis":
            return "reasoning"
        if self.channel == "final":
            return "final"
        return "commentary"


_TERMINATORS = (END, CALL, RETURN)


def _parse_header(header: str, msg: HarmonyMessage, default_role: str) -> None:
    role_part, _, chan_part = header.partition(CHANNEL)
    chan_part, _, ctype = chan_part.partition(CONSTRAIN)
    msg.content_type = ctype.strip() or None
    for part, is_role in ((role_part, True), (chan_part, False)):
        words = part.split()
        for w in words:
            if w.startswith("to="):
                msg.recipient = w[3:]
        plain = [w for w in words if not w.startswith("to=")]
        if is_role:
            msg.role = plain[0] if plain else default_role
        elif plain:
            msg.channel = plain[0]


def parse_harmony(text: str, default_role: str = "assistant") -> List[HarmonyMessage]:
    """Split harmony text into messages.  A completion starts inside the assistant message the prompt opened, so the
    first message may begin with ``<|channel|>`` (or with plain text when the model wrote no markers)."""
    out: List[HarmonyMessage] = []
    chunks = text.split(START)
    for n, chunk in enumerate(chunks):
        if n == 0 and not chunk:
            continue
        msg = HarmonyMessage(role=default_role)
        if MESSAGE in chunk:
            header, body = chunk.split(MESSAGE, 1)
            _parse_header(header, msg, default_role)
            cut, term = len(body), None
            for t in _TERMINATORS:
                k = body.find(t)
                if 0 <= k < cut:
                    cut, term = k, t
            msg.body, msg.terminator = body[:cut], term
        elif n == 0 and CHANNEL not in chunk:
            msg.body = chunk                             # bare text without markers
            for t in _TERMINATORS:
                if msg.body.endswith(t):
                    msg.body, msg.terminator = msg.body[: -len(t)], t
        else:
            _parse_header(chunk, msg, default_role)
            msg.header_complete = False
        out.append(msg)
    return out


def parse_completion(text: str) -> Dict[str, Any]:
    """Completion text -> reasoning (analysis channel), content (final channel, else commentary preambles or bare
    text) and OpenAI-format tool calls."""
    reasoning, finals, commentary, calls = [], [], [], []
    for m in parse_harmony(text):
        if not m.header_complete:
            continue
        if m.kind == "tool_call":
            calls.append({"id": f"call_{len(calls)}", "type": "function",
                          "function": {"name": m.recipient[len(NAMESPACE) + 1:], "arguments": m.body}})
        elif m.kind == "reasoning":
            reasoning.append(m.body)
        elif m.kind == "final":
            finals.append(m.body)
        else:
            commentary.append(m.body)
    content = "".join(finals) if finals else "".join(commentary)
    return {"role": "assistant", "reasoning_content": "\n".join(reasoning) if reasoning else None, "content": content,
            "tool_calls": calls}
