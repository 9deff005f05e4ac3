"""GPT-OSS harmony format: prompt rendering, tool declarations, completion parsing.  Where a checkout of the reference
sits beside this repository, the expected texts of its unit test (a table of JSON schemas and the declarations the
harmony reference renderer writes for them) are read as data and checked against this repository's renderer."""
import ast
import json
import os

import pytest

from batchgen_b200.runtime import harmony as H

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TEST = os.path.join(os.path.dirname(_REPO), "reference", "tests", "unit", "test_gpt_oss_chat_template.py")


def _tool(name, description, parameters=None, with_parameters=True):
    fn = {"name": name, "description": description}
    if with_parameters:
        fn["parameters"] = parameters
    return {"type": "function", "function": fn}


def _decl(parameters, description=""):
    text = H.render_functions_namespace([_tool("f", description, parameters)])
    head, tail = "# Tools\n\n## functions\n\nnamespace functions {\n\n", "\n\n} // namespace functions"
    assert text.startswith(head) and text.endswith(tail)
    return text[len(head):-len(tail)]


WEATHER = _tool("get_weather", "Get the weather.", {
    "type": "object",
    "properties": {"location": {"type": "string", "description": "City name"}, "unit": {"type": "string", "enum": ["c", "f"]},
                   "days": {"type": "integer", "description": "Forecast days", "default": 1},
                   "tags": {"type": "array", "items": {"type": "string"}}, "opt": {"type": ["string", "null"]},
                   "nested": {"type": "object", "properties": {"a": {"type": "string"}}}},
    "required": ["location"]})


def test_declarations_of_common_schemas():
    assert _decl(WEATHER["function"]["parameters"], "Get the weather.") == (
        "// Get the weather.\ntype f = (_: {\n// City name\nlocation: string,\n"
        'unit?: "c" | "f",\n// Forecast days\ndays?: number, // default: 1\ntags?: string[],\nopt?: string | null,\n'
        "nested?: {\n    a?: string,\n    },\n}) => any;")
    assert H.render_functions_namespace([_tool("no_args", "Takes nothing.", with_parameters=False)]).endswith(
        "// Takes nothing.\ntype no_args = () => any;\n\n} // namespace functions")
    assert _decl({}) == "type f = (_: any) => any;"
    assert _decl({"type": "object", "properties": {"a": {"type": "number", "default": 1e20}}}) == \
        "type f = (_: {\na?: number, // default: 1e20\n}) => any;"
    odd = {"oneOf": [{"type": "string"}, {"type": "number"}]}
    assert _decl({"type": "object", "properties": {"x": odd}, "required": ["x"]}) == \
        "type f = (_: {\n// JSON schema: " + json.dumps(odd) + "\nx: any,\n}) => any;"
    with pytest.raises(ValueError, match="duplicate function name"):
        H.render_functions_namespace([_tool("f", ""), _tool("f", "")])
    with pytest.raises(ValueError, match="contains whitespace"):
        H.render_functions_namespace([_tool("get weather", "")])


ARGS = '{"location": "Paris", "unit": "c"}'
TWO_TURN = [
    {"role": "system", "content": "Reasoning: low"},
    {"role": "user", "content": "Weather in Paris?"},
    {"role": "assistant", "content": "", "reasoning_content": "User asks weather. Use tool.",
     "tool_calls": [{"id": "call_1", "type": "function", "function": {"name": "get_weather", "arguments": ARGS}}]},
    {"role": "tool", "tool_call_id": "call_1", "content": '{"temp_c": 21}'},
]
CALL = "<|start|>assistant to=functions.get_weather<|channel|>commentary <|constrain|>json<|message|>" + ARGS + "<|call|>"
RESULT = '<|start|>functions.get_weather to=assistant<|channel|>commentary<|message|>{"temp_c": 21}<|end|>'


def test_prompt_without_and_with_tools():
    plain = H.render_harmony_prompt([{"role": "system", "content": "Reasoning: low\nBe brief."}, {"role": "user", "content": "hi"},
                                     {"role": "assistant", "content": "hello"}, {"role": "user", "content": "bye"}],
                                    add_generation_prompt=True)
    assert plain == ("<|start|>system<|message|>Reasoning: low\nBe brief." + H.SYSTEM_SUFFIX + "<|end|>"
                     "<|start|>user<|message|>hi<|end|><|start|>assistant<|channel|>final<|message|>hello<|end|>"
                     "<|start|>user<|message|>bye<|end|><|start|>assistant")
    rendered = H.render_harmony_prompt(TWO_TURN, tools=[WEATHER], add_generation_prompt=True)
    assert rendered == (
        "<|start|>system<|message|>Reasoning: low" + H.SYSTEM_SUFFIX + H.TOOL_NOTE + "<|end|>"
        "<|start|>developer<|message|>" + H.render_functions_namespace([WEATHER]) + "<|end|>"
        "<|start|>user<|message|>Weather in Paris?<|end|>"
        "<|start|>assistant<|channel|>analysis<|message|>User asks weather. Use tool.<|end|>" + CALL + RESULT + "<|start|>assistant")
    finished = TWO_TURN + [{"role": "assistant", "content": "It is 21 C.", "reasoning_content": "Answer."},
                           {"role": "user", "content": "And Rome?"}]
    later = H.render_harmony_prompt(finished, tools=[WEATHER], add_generation_prompt=True)
    assert "<|channel|>analysis" not in later                 # reasoning of a finished turn is dropped
    no_system = H.render_harmony_prompt([{"role": "user", "content": "q"}], tools=[WEATHER])
    assert no_system.startswith("<|start|>developer<|message|># Tools") and H.TOOL_NOTE not in no_system


@pytest.mark.parametrize("messages,needle", [
    ([{"role": "tool", "tool_call_id": "nope", "content": "x"}], "matches no earlier assistant tool call"),
    ([{"role": "tool", "content": "x"}], "needs tool_call_id (or name)"),
    ([{"role": "developer", "content": "x"}], "role 'developer' is not supported"),
    ([{"role": "user"}], "'content' must be a string"),
    ([{"role": "assistant", "tool_calls": [{"id": "a", "function": {"name": "f", "arguments": {"x": 1}}}]}],
     "function.arguments must be the JSON-encoded string"),
])
def test_conversations_the_format_cannot_carry_are_refused(messages, needle):
    with pytest.raises(ValueError) as e:
        H.render_harmony_prompt(messages)
    assert needle in str(e.value)


def test_completion_parsing_and_round_trip_through_history():
    completion = ("<|channel|>analysis<|message|>User asks weather. Use tool.<|end|>"
                  "<|start|>assistant<|channel|>commentary to=functions.get_weather <|constrain|>json<|message|>" + ARGS + "<|call|>")
    parsed = H.parse_completion(completion)
    assert parsed["reasoning_content"] == "User asks weather. Use tool." and parsed["content"] == ""
    assert parsed["tool_calls"][0]["function"] == {"name": "get_weather", "arguments": ARGS}
    turn2 = TWO_TURN[:2] + [dict(parsed), {"role": "tool", "tool_call_id": parsed["tool_calls"][0]["id"], "content": '{"temp_c": 21}'}]
    assert H.render_harmony_prompt(turn2, tools=[WEATHER], add_generation_prompt=True) == \
        H.render_harmony_prompt(TWO_TURN, tools=[WEATHER], add_generation_prompt=True)
    (call,) = H.parse_harmony(CALL)
    assert call.kind == "tool_call" and call.recipient == "functions.get_weather" and call.content_type == "json"
    (res,) = H.parse_harmony(RESULT)
    assert (res.role, res.recipient, res.channel, res.body) == ("functions.get_weather", "assistant", "commentary", '{"temp_c": 21}')
    final = H.parse_completion("<|channel|>analysis<|message|>think<|end|><|start|>assistant<|channel|>final<|message|>42<|return|>")
    assert final["reasoning_content"] == "think" and final["content"] == "42" and final["tool_calls"] == []
    assert H.parse_completion("just text")["content"] == "just text"
    history = H.parse_harmony(CALL + RESULT + "<|start|>assistant")
    assert len(history) == 3 and not history[-1].header_complete


def _reference_tables():
    """SUPPORTED_SCHEMAS / EXOTIC_PROPERTY_SCHEMAS / WEATHER_NAMESPACE literals of the reference's unit test."""
    tree = ast.parse(open(REF_TEST, encoding="utf-8").read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            if node.targets[0].id in ("SUPPORTED_SCHEMAS", "EXOTIC_PROPERTY_SCHEMAS", "WEATHER_NAMESPACE"):
                out[node.targets[0].id] = ast.literal_eval(node.value)
    return out


@pytest.mark.skipif(not os.path.isfile(REF_TEST), reason="reference checkout not present")
def test_declarations_match_the_reference_renderer_tables():
    tables = _reference_tables()
    assert len(tables["SUPPORTED_SCHEMAS"]) >= 20
    for case, (schema, expected) in tables["SUPPORTED_SCHEMAS"].items():
        assert _decl(schema) == expected, case
    for case, schema in tables["EXOTIC_PROPERTY_SCHEMAS"].items():
        got = _decl({"type": "object", "properties": {"ok": {"type": "string"}, "x": schema}, "required": ["x"]})
        want = "type f = (_: {\nok?: string,\n// JSON schema: " + json.dumps(schema, ensure_ascii=False) + "\nx: any,\n}) => any;"
        assert got == want, case
    full = dict(WEATHER["function"]["parameters"])
    full["properties"] = {"location": {"type": "string", "description": "City name"}, "unit": {"type": "string", "enum": ["c", "f"]},
                          "days": {"type": "integer", "description": "Forecast days", "default": 1}, "precise": {"type": "boolean"},
                          "ratio": {"type": "number"}, "tags": {"type": "array", "items": {"type": "string"}},
                          "nums": {"type": "array", "items": {"type": "integer"}}, "opt": {"type": ["string", "null"]},
                          "nested": {"type": "object", "properties": {"a": {"type": "string"}}}}
    tools = [_tool("get_weather", "Get the weather.", full), _tool("no_args", "Takes nothing.", with_parameters=False),
             _tool("empty_obj", "Empty object.", {"type": "object", "properties": {}})]
    assert H.render_functions_namespace(tools) == tables["WEATHER_NAMESPACE"]


def test_chat_requests_of_a_gpt_oss_model_use_harmony_end_to_end():
    from batchgen_b200.runtime.batch_api import BatchOptions, BatchRequest, prompt_ids, result_item
    from batchgen_b200.runtime.sequence import Sequence
    from batchgen_b200.runtime.tokenization import get_tokenizer
    tok = get_tokenizer("bytes", 512, chat_format="harmony")
    body = {"messages": [{"role": "user", "content": "Weather in Paris?"}], "tools": [WEATHER], "reasoning_effort": "low",
            "max_tokens": 8}
    req = BatchRequest(custom_id="r1", url="/v1/chat/completions", body=body)
    text = tok.decode(prompt_ids(req, tok))
    assert text.startswith("<|start|>system<|message|>Reasoning: low" + H.SYSTEM_SUFFIX + H.TOOL_NOTE + "<|end|><|start|>developer")
    assert text.endswith("<|start|>user<|message|>Weather in Paris?<|end|><|start|>assistant")
    seq = Sequence(0, [1, 2, 3])
    seq.output_ids = tok.encode("<|channel|>analysis<|message|>need the tool<|end|><|start|>assistant<|channel|>commentary "
                                "to=functions.get_weather <|constrain|>json<|message|>" + ARGS + "<|call|>")
    seq.finish_reason = "stop"
    item = result_item(seq, req, tok, BatchOptions(model="tiny-gpt-oss", parse_thinking=True, parse_tool_call=True))
    msg = item["response"]["body"]["choices"][0]["message"]
    assert msg["reasoning_content"] == "need the tool" and msg["content"] == ""
    assert msg["tool_calls"][0]["function"] == {"name": "get_weather", "arguments": ARGS}
