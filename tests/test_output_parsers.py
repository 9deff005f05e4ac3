"""Tool-call markup of each model family -> OpenAI tool_calls."""
import json

from batchgen_b200.runtime.output_parsers import FAMILY_FORMAT, parse_tool_calls


def _fn(calls):
    return [(c["function"]["name"], json.loads(c["function"]["arguments"])) for c in calls]


def test_json_format_is_the_default():
    calls, rest = parse_tool_calls('Let me check.\n<tool_call>\n{"name": "get", "arguments": {"city": "Paris"}}\n</tool_call>')
    assert _fn(calls) == [("get", {"city": "Paris"})] and rest == "Let me check."
    assert parse_tool_calls("no calls here") == ([], "no calls here")
    assert parse_tool_calls("<tool_call>{broken</tool_call>")[0] == []


def test_glm_key_value_markup():
    text = ("I will look it up.<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Beijing</arg_value>\n"
            "<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n<arg_key>opts</arg_key><arg_value>{\"u\": \"c\"}</arg_value>\n</tool_call>"
            "<tool_call>now</tool_call>")
    calls, rest = parse_tool_calls(text, "glm")
    assert _fn(calls) == [("get_weather", {"city": "Beijing", "days": 3, "opts": {"u": "c"}}), ("now", {})]
    assert rest == "I will look it up."


def test_kimi_sections_keep_the_models_call_ids():
    text = ("ok<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>"
            '{"city": "Beijing"}<|tool_call_end|><|tool_call_begin|>functions.search:1<|tool_call_argument_begin|>'
            '{"q": "x"}<|tool_call_end|><|tool_calls_section_end|>')
    calls, rest = parse_tool_calls(text, "kimi")
    assert _fn(calls) == [("get_weather", {"city": "Beijing"}), ("search", {"q": "x"})]
    assert [c["id"] for c in calls] == ["functions.get_weather:0", "functions.search:1"] and rest == "ok"


def test_minimax_invoke_blocks():
    text = ('<minimax:tool_call>\n<invoke name="get_weather">\n<parameter name="city">SF</parameter>\n'
            '<parameter name="days">2</parameter>\n</invoke>\n<invoke name="ping">\n</invoke>\n</minimax:tool_call>done')
    calls, rest = parse_tool_calls(text, "minimax")
    assert _fn(calls) == [("get_weather", {"city": "SF", "days": 2}), ("ping", {})] and rest == "done"


def test_deepseek_both_generations_of_the_markup():
    new = ('<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>get_weather<｜tool▁sep｜>{"city": "Hangzhou"}<｜tool▁call▁end｜>'
           '<｜tool▁call▁begin｜>get_time<｜tool▁sep｜>{}<｜tool▁call▁end｜><｜tool▁calls▁end｜>')
    calls, rest = parse_tool_calls("Sure. " + new, "deepseek")
    assert _fn(calls) == [("get_weather", {"city": "Hangzhou"}), ("get_time", {})] and rest == "Sure."
    old = ('<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n{"city": "Hangzhou"}\n```'
           '<｜tool▁call▁end｜><｜tool▁calls▁end｜>')
    calls, rest = parse_tool_calls(old, "deepseek")
    assert _fn(calls) == [("get_weather", {"city": "Hangzhou"})] and rest == ""


def test_family_table_and_batch_api_hook():
    assert FAMILY_FORMAT["glm5"] == "glm" and FAMILY_FORMAT["kimi_k3"] == "kimi" and FAMILY_FORMAT["deepseek_v3"] == "deepseek"
    from batchgen_b200.runtime.batch_api import BatchOptions, BatchRequest, result_item
    from batchgen_b200.runtime.sequence import Sequence
    from batchgen_b200.runtime.tokenization import get_tokenizer
    tok = get_tokenizer("bytes", 512)
    seq = Sequence(0, [1, 2, 3])
    seq.output_ids = tok.encode("<think>use the tool</think><tool_call>lookup<arg_key>k</arg_key><arg_value>v</arg_value></tool_call>")
    seq.finish_reason = "stop"
    req = BatchRequest(custom_id="r", url="/v1/chat/completions", body={"messages": [], "max_tokens": 4})
    item = result_item(seq, req, tok, BatchOptions(parse_thinking=True, parse_tool_call=True, tool_call_format="glm"))
    msg = item["response"]["body"]["choices"][0]["message"]
    assert msg["reasoning_content"] == "use the tool" and msg["content"] == ""
    assert _fn(msg["tool_calls"]) == [("lookup", {"k": "v"})]


def test_audit_of_an_output_file(tmp_path):
    from batchgen_b200.runtime.output_parsers import audit_output_file
    def item(text):
        return {"custom_id": "x", "response": {"body": {"choices": [{"message": {"content": text}}]}}}
    texts = ["plain answer", "<tool_call>f<arg_key>a</arg_key><arg_value>1</arg_value></tool_call>",
             "<tool_call>g</tool_call><tool_call>h</tool_call>", "broken <tool_call>never closed"]
    p = tmp_path / "out.jsonl"
    p.write_text("\n".join(json.dumps(item(t)) for t in texts) + "\n")
    assert audit_output_file(str(p), "glm") == {"items": 4, "with_calls": 2, "calls": 3, "bad_arguments": 0, "leftover_markup": 1}
