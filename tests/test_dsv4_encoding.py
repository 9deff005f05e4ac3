"""DeepSeek-V4 prompt encoding: the published format's cases, and its golden prompt files where the reference tree is
present (they are read as text; the encoder under test is this repository's own)."""
import json
import os

import pytest

from batchgen_b200.runtime import dsv4_encoding as enc

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(os.path.dirname(_REPO), "reference", "batchgen", "models", "deepseek", "deepseekv4_flash", "assets",
                    "encoding", "tests")          # a checkout of the reference beside this repository, when there is one
needs_gold = pytest.mark.skipif(not os.path.isdir(GOLD), reason="golden prompt files not present")


def _load(n):
    data = json.load(open(os.path.join(GOLD, f"test_input_{n}.json"), encoding="utf-8"))
    gold = open(os.path.join(GOLD, f"test_output_{n}.txt"), encoding="utf-8").read()
    return data, gold


def test_basic_thinking_and_chat_prompts():
    msgs = [{"role": "system", "content": "You are a helpful assistant."}, {"role": "user", "content": "What is 2+2?"}]
    assert enc.encode_messages(msgs, "thinking") == (
        "<｜begin▁of▁sentence｜>You are a helpful assistant.<｜User｜>What is 2+2?<｜Assistant｜><think>")
    assert enc.encode_messages(msgs, "chat").endswith("<｜Assistant｜></think>")
    parsed = enc.parse_completion("Simple arithmetic.</think>2 + 2 = 4.<｜end▁of▁sentence｜>", "thinking")
    assert parsed == {"role": "assistant", "reasoning_content": "Simple arithmetic.", "content": "2 + 2 = 4.", "tool_calls": []}
    assert enc.parse_completion("4<｜end▁of▁sentence｜>", "chat")["content"] == "4"
    assert enc.encode_messages(msgs, "thinking", reasoning_effort="max").startswith(enc.BOS + "Reasoning Effort: Absolute maximum")
    with pytest.raises(ValueError):
        enc.encode_messages(msgs, "fast")


def test_reasoning_of_earlier_turns_is_dropped_without_tools_and_kept_with_tools():
    msgs = [{"role": "user", "content": "a"}, {"role": "assistant", "reasoning_content": "r1", "content": "b"},
            {"role": "user", "content": "c"}, {"role": "assistant", "reasoning_content": "r2", "content": "d"}]
    p = enc.encode_messages(msgs, "thinking")
    assert "r1" not in p and "<think>r2</think>d" in p and "<｜Assistant｜></think>b" in p
    assert "r1" in enc.encode_messages(msgs, "thinking", drop_thinking=False)
    tools = [{"type": "function", "function": {"name": "f", "parameters": {}}}]
    with_tools = [{"role": "system", "content": "s", "tools": tools}] + msgs
    assert "<think>r1</think>b" in enc.encode_messages(with_tools, "thinking")
    assert "r1" not in enc.encode_messages(msgs, "chat") and "r2" not in enc.encode_messages(msgs, "chat")


def test_tool_calls_round_trip_and_results_follow_call_order():
    calls = [{"id": "x", "type": "function", "function": {"name": "get", "arguments": json.dumps({"city": "Paris", "days": 3, "opts": {"u": "c"}})}},
             {"id": "y", "type": "function", "function": {"name": "find", "arguments": "{\"q\": \"a b\"}"}}]
    block = enc.render_tool_calls(calls)
    assert '<｜DSML｜parameter name="city" string="true">Paris</｜DSML｜parameter>' in block
    assert '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>' in block
    parsed = enc.parse_completion("think</think>\n\n" + block + enc.EOS, "thinking")
    assert parsed["content"] == "" and [c["function"]["name"] for c in parsed["tool_calls"]] == ["get", "find"]
    assert json.loads(parsed["tool_calls"][0]["function"]["arguments"]) == {"city": "Paris", "days": 3, "opts": {"u": "c"}}
    msgs = [{"role": "user", "content": "q"}, {"role": "assistant", "content": "", "tool_calls": calls},
            {"role": "tool", "tool_call_id": "y", "content": "second"}, {"role": "tool", "tool_call_id": "x", "content": "first"}]
    p = enc.encode_messages(msgs, "thinking")
    assert p.index("<tool_result>first</tool_result>") < p.index("<tool_result>second</tool_result>")
    assert p.count("<｜User｜>") == 2 and p.endswith("<｜Assistant｜><think>")


def test_task_tokens():
    assert enc.encode_messages([{"role": "user", "content": "q", "task": "query"}], "chat").endswith("<｜User｜>q<｜query｜>")
    assert enc.encode_messages([{"role": "user", "content": "q", "task": "action"}], "thinking").endswith("<｜Assistant｜><think><｜action｜>")
    p = enc.encode_messages([{"role": "user", "content": "q"}, {"role": "assistant", "content": "a", "task": "title"},
                             {"role": "assistant", "content": "A title"}], "chat")
    assert p.endswith("a<｜end▁of▁sentence｜><｜title｜>A title<｜end▁of▁sentence｜>")


@needs_gold
def test_golden_thinking_with_tools():
    data, gold = _load(1)
    msgs = data["messages"]
    msgs[0]["tools"] = data["tools"]
    prompt = enc.encode_messages(msgs, "thinking")
    assert prompt == gold
    marker = "<｜Assistant｜><think>"
    a = prompt.find(marker) + len(marker)
    first = enc.parse_completion(prompt[a: prompt.find("<｜User｜>", a)], "thinking")
    assert first["content"] == "" and first["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(first["tool_calls"][0]["function"]["arguments"]) == {"location": "Beijing", "unit": "celsius"}
    last = enc.parse_completion(prompt[prompt.rfind(marker) + len(marker):], "thinking")
    assert last["reasoning_content"].startswith("Got the weather data") and "22°C" in last["content"] and last["tool_calls"] == []


@needs_gold
@pytest.mark.parametrize("n,mode", [(2, "thinking"), (3, "thinking"), (4, "chat")])
def test_golden_prompts(n, mode):
    msgs, gold = _load(n)
    assert enc.encode_messages(msgs, mode) == gold


def test_chat_requests_of_a_v4_model_use_the_format_end_to_end():
    """Byte tokenizer + DeepSeek-V4 chat format: the prompt ids decode to the rendered prompt, and a completion in the
    family's format is split into reasoning, content and tool calls by the batch API."""
    from batchgen_b200.runtime.batch_api import BatchOptions, BatchRequest, prompt_ids, result_item
    from batchgen_b200.runtime.sequence import Sequence
    from batchgen_b200.runtime.tokenization import get_tokenizer
    tok = get_tokenizer("bytes", 512, chat_format="deepseek_v4")
    tools = [{"type": "function", "function": {"name": "get", "parameters": {"type": "object"}}}]
    body = {"messages": [{"role": "user", "content": "hi"}], "tools": tools, "max_tokens": 8}
    req = BatchRequest(custom_id="r1", url="/v1/chat/completions", body=body)
    ids = prompt_ids(req, tok)
    text = tok.decode(ids)
    assert text.startswith(enc.BOS) and "## Tools" in text and text.endswith("<｜User｜>hi<｜Assistant｜><think>")
    completion = "need the tool</think>\n\n" + enc.render_tool_calls([{"function": {"name": "get", "arguments": {"k": 1}}}]) + enc.EOS
    seq = Sequence(0, ids)
    seq.output_ids = tok.encode(completion)
    seq.finish_reason = "stop"
    item = result_item(seq, req, tok, BatchOptions(model="tiny-deepseek-v4", parse_thinking=True, parse_tool_call=True))
    msg = item["response"]["body"]["choices"][0]["message"]
    assert msg["reasoning_content"] == "need the tool" and msg["content"] == ""
    assert msg["tool_calls"][0]["function"]["name"] == "get" and json.loads(msg["tool_calls"][0]["function"]["arguments"]) == {"k": 1}
