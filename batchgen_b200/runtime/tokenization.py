"""Tokenisers and chat templating for the batch front end.

No tokenizer files ship with this repository (and none can be downloaded), so three tokenisers are
built in, selected by name or path:

* ``ids``   — prompts are token ids (a JSON list, or a string of space separated integers); used by
              the synthetic benchmarks.
* ``bytes`` — UTF-8 bytes shifted past the special ids; works for any vocabulary >= 259.
* a path    — a local Hugging Face ``tokenizer.json`` directory, loaded with ``transformers`` when present
              (the reference bundles per-model ``tokenizer.json`` files and Jinja chat templates:
              batchgen/tokenization.py:30-244, batchgen/config/fast_tokenizer.py:88,306-330).

``apply_chat_template`` renders ``messages`` with the tokenizer's own Jinja template when it has one and
with a plain role-tagged fallback otherwise; ``split_reasoning`` separates ``<think>...</think>`` content
for ``--parse-thinking``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple, Union


class IdTokenizer:
    name = "ids"

    def __init__(self, vocab_size: int, bos: int = 0, eos: int = 1):
        self.vocab_size, self.bos_token_id, self.eos_token_id = vocab_size, bos, eos

    def encode(self, text: Union[str, Sequence[int]]) -> List[int]:
        if isinstance(text, str):
            ids = [int(t) for t in text.replace(",", " ").split()] if text.strip() else []
        else:
            ids = [int(t) for t in text]
        for t in ids:
            if not 0 <= t < self.vocab_size:
                raise ValueError(f"token id {t} outside the vocabulary [0, {self.vocab_size})")
        return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return " ".join(str(int(i)) for i in ids)

    def apply_chat_template(self, messages: List[Dict], **kw) -> List[int]:
        out: List[int] = []
        for m in messages:
            c = m.get("content", "")
            out += self.encode(c if isinstance(c, (str, list)) else str(c))
        return out


class ByteTokenizer:
    name = "bytes"
    OFFSET = 3

    def __init__(self, vocab_size: int, bos: int = 0, eos: int = 1):
        if vocab_size < 256 + self.OFFSET:
            raise ValueError("the byte tokenizer needs a vocabulary of at least 259")
        self.vocab_size, self.bos_token_id, self.eos_token_id = vocab_size, bos, eos

    def encode(self, text: str) -> List[int]:
        return [b + self.OFFSET for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        bs = bytes(i - self.OFFSET for i in ids if self.OFFSET <= i < 256 + self.OFFSET)
        return bs.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages: List[Dict], add_generation_prompt: bool = True, **kw) -> List[int]:
        return self.encode(render_fallback_template(messages, add_generation_prompt))


class HFTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(path, local_files_only=True)
        self.name = path
        self.vocab_size = len(self.tok)
        self.bos_token_id, self.eos_token_id = self.tok.bos_token_id, self.tok.eos_token_id

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def apply_chat_template(self, messages: List[Dict], add_generation_prompt: bool = True, **kw) -> List[int]:
        if getattr(self.tok, "chat_template", None):
            return self.tok.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
        return self.encode(render_fallback_template(messages, add_generation_prompt))


def render_fallback_template(messages: List[Dict], add_generation_prompt: bool = True) -> str:
    parts = []
    for m in messages:
        role, content = m.get("role", "user"), m.get("content", "")
        if isinstance(content, list):            # OpenAI content parts: keep the text ones
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
        parts.append(f"<|{role}|>\n{content}\n")
    if add_generation_prompt:
        parts.append("<|assistant|>\n")
    return "".join(parts)


class DeepSeekV4Chat:
    """A tokenizer whose chat rendering and completion parsing follow the DeepSeek-V4 format (``runtime.dsv4_encoding``:
    the family ships no Jinja template).  ``enable_thinking`` selects thinking or chat mode, ``tools`` are attached to
    the system message (one is created when the conversation has none)."""

    def __init__(self, base):
        self.base = base
        self.name = f"{getattr(base, 'name', 'tokenizer')}+deepseek_v4"
        self.vocab_size, self.bos_token_id, self.eos_token_id = base.vocab_size, base.bos_token_id, base.eos_token_id

    def encode(self, text):
        return self.base.encode(text)

    def decode(self, ids, skip_special_tokens: bool = True):
        return self.base.decode(ids, skip_special_tokens=skip_special_tokens)

    def render(self, messages: List[Dict], enable_thinking: bool = True, reasoning_effort: Optional[str] = None,
               tools: Optional[List[Dict]] = None) -> str:
        from . import dsv4_encoding
        msgs = [dict(m) for m in messages]
        if tools:
            holder = next((m for m in msgs if m.get("role") in ("system", "developer")), None)
            if holder is None:
                holder = {"role": "system", "content": ""}
                msgs.insert(0, holder)
            holder["tools"] = list(tools)
        return dsv4_encoding.encode_messages(msgs, "thinking" if enable_thinking else "chat",
                                             reasoning_effort=reasoning_effort)

    def apply_chat_template(self, messages: List[Dict], add_generation_prompt: bool = True, enable_thinking: bool = True,
                            reasoning_effort: Optional[str] = None, tools: Optional[List[Dict]] = None, **kw) -> List[int]:
        self._thinking = bool(enable_thinking)
        return self.encode(self.render(messages, enable_thinking, reasoning_effort, tools))

    def parse_completion(self, text: str, enable_thinking: bool = True) -> Dict:
        from . import dsv4_encoding
        return dsv4_encoding.parse_completion(text, "thinking" if enable_thinking else "chat")


class HarmonyChat:
    """A tokenizer whose chat rendering and completion parsing follow the GPT-OSS harmony format
    (``runtime.harmony``): tools become the developer message's ``functions`` namespace, tool-call history and tool
    results become call / result messages, completions are split by channel.  ``reasoning_effort`` is written as the
    system message's ``Reasoning:`` line when the conversation does not set one itself."""

    def __init__(self, base):
        self.base = base
        self.name = f"{getattr(base, 'name', 'tokenizer')}+harmony"
        self.vocab_size, self.bos_token_id, self.eos_token_id = base.vocab_size, base.bos_token_id, base.eos_token_id

    def encode(self, text):
        return self.base.encode(text)

    def decode(self, ids, skip_special_tokens: bool = True):
        return self.base.decode(ids, skip_special_tokens=skip_special_tokens)

    def render(self, messages: List[Dict], add_generation_prompt: bool = True, reasoning_effort: Optional[str] = None,
               tools: Optional[List[Dict]] = None) -> str:
        from . import harmony
        msgs = [dict(m) for m in messages]
        if reasoning_effort:
            line = f"Reasoning: {reasoning_effort}"
            if msgs and msgs[0].get("role") == "system":
                if "Reasoning:" not in (msgs[0].get("content") or ""):
                    msgs[0]["content"] = line + ("\n" + msgs[0]["content"] if msgs[0].get("content") else "")
            else:
                msgs.insert(0, {"role": "system", "content": line})
        return harmony.render_harmony_prompt(msgs, tools=tools or None, add_generation_prompt=add_generation_prompt)

    def apply_chat_template(self, messages: List[Dict], add_generation_prompt: bool = True,
                            reasoning_effort: Optional[str] = None, tools: Optional[List[Dict]] = None, **kw) -> List[int]:
        return self.encode(self.render(messages, add_generation_prompt, reasoning_effort, tools))

    def parse_completion(self, text: str, enable_thinking: bool = True) -> Dict:
        from . import harmony
        return harmony.parse_completion(text)


def chat_format_for(family: str) -> Optional[str]:
    """The Python-rendered chat format of a model family (None: the tokenizer's own template)."""
    return {"deepseek_v4": "deepseek_v4", "gpt_oss": "harmony"}.get(family)


def get_tokenizer(spec: str, vocab_size: int, bos: int = 0, eos: int = 1, chat_format: Optional[str] = None):
    """``chat_format`` ("deepseek_v4" or "harmony") wraps the tokenizer so that chat requests use that family's
    prompt format and completion parser."""
    if spec in ("ids", "", None):
        tok = IdTokenizer(vocab_size, bos, eos)
    elif spec == "bytes":
        tok = ByteTokenizer(vocab_size, bos, eos)
    elif os.path.isdir(spec):
        tok = HFTokenizer(spec)
    else:
        raise ValueError(f"unknown tokenizer {spec!r}: use 'ids', 'bytes' or a local tokenizer directory")
    if chat_format not in (None, "", "deepseek_v4", "harmony"):
        raise ValueError(f"unknown chat format {chat_format!r}")
    if chat_format and not isinstance(tok, IdTokenizer):          # the id tokenizer has no text to render into
        return DeepSeekV4Chat(tok) if chat_format == "deepseek_v4" else HarmonyChat(tok)
    return tok


_THINK = re.compile(r"<think>(.*?)</think>", re.S)


def split_reasoning(text: str) -> Tuple[Optional[str], str]:
    """-> (reasoning_content or None, content) for ``<think>...</think>`` style outputs."""
    m = _THINK.search(text)
    if not m:
        if "</think>" in text:                      # template opened the block in the prompt
            r, c = text.split("</think>", 1)
            return r.strip(), c.strip()
        return None, text
    return m.group(1).strip(), (text[: m.start()] + text[m.end():]).strip()


_TOOL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str) -> Tuple[List[Dict], str]:
    """Extract ``<tool_call>{json}</tool_call>`` blocks -> (OpenAI tool_calls list, remaining text)."""
    calls = []
    for i, m in enumerate(_TOOL.finditer(text)):
        try:
            obj = json.loads(m.group(1))
        except ValueError:
            continue
        calls.append({"id": f"call_{i}", "type": "function",
                      "function": {"name": obj.get("name", ""), "arguments": json.dumps(obj.get("arguments", {}))}})
    return calls, _TOOL.sub("", text).strip()
