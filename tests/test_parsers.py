"""Tool-call and reasoning parsers of the chat endpoint, and the OpenAI ``logprobs`` objects."""
import json

import pytest

from vllm_metax_b200.entrypoints.openai_server import format_logprobs
from vllm_metax_b200.entrypoints.parsers import (get_reasoning_parser, get_tool_parser, parse_chat_output,
                                                 parse_deepseek_v3, parse_hermes, parse_llama3_json, parse_mistral,
                                                 parse_pythonic, split_think)


def _args(call):
    return json.loads(call.arguments)


def test_hermes_calls_and_surrounding_text():
    text = ('Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>\n'
            '<tool_call>{"name": "get_time", "arguments": {"tz": "CET"}}</tool_call>')
    m = parse_hermes(text)
    assert [c.name for c in m.tool_calls] == ["get_weather", "get_time"]
    assert _args(m.tool_calls[0]) == {"city": "Paris"} and m.content == "Let me check."
    assert parse_hermes("plain answer").tool_calls == [] and parse_hermes("plain answer").content == "plain answer"
    # a call cut off by max_tokens still parses when its JSON is complete
    assert parse_hermes('<tool_call>{"name": "f", "arguments": {}}').tool_calls[0].name == "f"
    assert parse_hermes('<tool_call>{"name": "f", "argu').tool_calls == []


def test_llama3_json_mistral_deepseek_pythonic():
    m = parse_llama3_json('<|python_tag|>{"name": "add", "parameters": {"a": 1, "b": 2}}; {"name": "neg", "parameters": {"x": 3}}')
    assert [c.name for c in m.tool_calls] == ["add", "neg"] and _args(m.tool_calls[0]) == {"a": 1, "b": 2}
    assert parse_llama3_json("The answer is {not json}").tool_calls == []
    assert parse_llama3_json('{"temperature": 3}').tool_calls == []            # JSON, but not a call
    m = parse_mistral('[TOOL_CALLS] [{"name": "search", "arguments": {"q": "b200"}}]')
    assert m.tool_calls[0].name == "search" and m.content is None
    ds = ("I will look it up.<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>lookup\n```json\n"
          '{"key": "v"}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>')
    m = parse_deepseek_v3(ds)
    assert m.tool_calls[0].name == "lookup" and _args(m.tool_calls[0]) == {"key": "v"} and m.content == "I will look it up."
    m = parse_pythonic('[get_weather(city="Paris", days=2), ping()]')
    assert [c.name for c in m.tool_calls] == ["get_weather", "ping"] and _args(m.tool_calls[0]) == {"city": "Paris", "days": 2}
    assert parse_pythonic("[1, 2, 3]").tool_calls == [] and parse_pythonic("[f(__import__('os'))]").tool_calls == []


def test_reasoning_split_and_combined_output():
    assert split_think("<think>step 1\nstep 2</think>\n\n42") == ("step 1\nstep 2", "42")
    assert split_think("step 1</think>42") == ("step 1", "42")                  # the template opened the tag
    assert split_think("no tags at all") == (None, "no tags at all")
    assert split_think("<think>still thinking") == ("still thinking", None)
    assert split_think("partial", finished=False) == ("partial", None)
    msg = parse_chat_output('<think>need the tool</think><tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>',
                            get_tool_parser("hermes"), get_reasoning_parser("deepseek_r1"), tools_requested=True)
    assert msg.reasoning_content == "need the tool" and msg.tool_calls[0].name == "f" and msg.content is None
    # without tools in the request the markup stays content
    msg = parse_chat_output('<tool_call>{"name": "f", "arguments": {}}</tool_call>', get_tool_parser("hermes"), None, False)
    assert msg.tool_calls == [] and msg.content.startswith("<tool_call>")
    # tool_choice named a function: the constrained answer is its arguments
    msg = parse_chat_output('{"city": "Rome"}', None, None, True, forced_tool="get_weather")
    assert msg.tool_calls[0].name == "get_weather" and json.loads(msg.tool_calls[0].arguments) == {"city": "Rome"}
    d = msg.tool_calls[0].to_openai(0)
    assert d["type"] == "function" and d["index"] == 0 and d["id"].startswith("call_")


def test_logprobs_objects():
    class Tok:
        def decode(self, ids):
            return "".join("ab"[i % 2] * (1 + i % 3) for i in ids)

    entries = [{"token_id": 1, "logprob": -0.5, "top": [(1, -0.5), (4, -1.5)]},
               {"token_id": 2, "logprob": -1.0, "top": [(3, -0.7), (2, -1.0)]}]
    c = format_logprobs(entries, Tok(), chat=False)
    assert c["tokens"] == ["bb", "aaa"] and c["text_offset"] == [0, 2] and c["token_logprobs"] == [-0.5, -1.0]
    assert c["top_logprobs"][1] == {"bb": -0.7, "aaa": -1.0} or len(c["top_logprobs"][1]) == 2
    ch = format_logprobs(entries, Tok(), chat=True, start=1)
    assert len(ch["content"]) == 1 and ch["content"][0]["token"] == "aaa" and len(ch["content"][0]["top_logprobs"]) == 2
    assert format_logprobs(None, Tok(), chat=True) is None


@pytest.mark.parametrize("name,text,want", [
    ("deepseek_v31", 'ok<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>get_weather<｜tool▁sep｜>{"city": "Paris"}<｜tool▁call▁end｜>'
                     '<｜tool▁call▁begin｜>add<｜tool▁sep｜>{"a": 1, "b": 2}<｜tool▁call▁end｜><｜tool▁calls▁end｜>',
     [("get_weather", {"city": "Paris"}), ("add", {"a": 1, "b": 2})]),
    ("granite", '<|tool_call|>[{"name": "get_weather", "arguments": {"city": "Paris"}}]', [("get_weather", {"city": "Paris"})]),
    ("granite-20b-fc", '<function_call> {"name": "f", "arguments": {"x": 1}}\n<function_call> {"name": "g", "arguments": {}}',
     [("f", {"x": 1}), ("g", {})]),
    ("phi4_mini_json", 'functools[{"name": "f", "arguments": {"x": [1, 2]}}]', [("f", {"x": [1, 2]})]),
    ("minimax", 'thinking\n<tool_calls>\n{"name": "f", "arguments": {"x": 1}}\n{"name": "g", "arguments": {"y": "z"}}\n</tool_calls>',
     [("f", {"x": 1}), ("g", {"y": "z"})]),
    ("hunyuan_a13b", '<tool_calls>[{"name": "f", "arguments": {"x": 1}}]</tool_calls>', [("f", {"x": 1})]),
    ("internlm", 'Let me check.<|action_start|><|plugin|>\n{"name": "f", "parameters": {"q": "a b"}}<|action_end|>',
     [("f", {"q": "a b"})]),
    ("xlam", '```json\n[{"name": "f", "arguments": {"x": 1}}]\n```', [("f", {"x": 1})]),
    ("xlam", '<think>hm</think>[{"name": "f", "arguments": {"x": 1}}]', [("f", {"x": 1})]),
    ("kimi_k2", '<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>'
                '{"city": "Paris"}<|tool_call_end|><|tool_calls_section_end|>', [("get_weather", {"city": "Paris"})]),
    ("qwen3_coder", 'Sure.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n'
                    '</parameter>\n</function>\n</tool_call>', [("get_weather", {"city": "Paris", "days": 3})]),
    ("glm45", '<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>metric</arg_key>\n'
              '<arg_value>true</arg_value>\n</tool_call>', [("get_weather", {"city": "Paris", "metric": True})]),
])
def test_more_tool_formats(name, text, want):
    import json as _json

    from vllm_metax_b200.entrypoints.parsers import get_tool_parser

    msg = get_tool_parser(name)(text)
    assert [(c.name, _json.loads(c.arguments)) for c in msg.tool_calls] == want
    plain = get_tool_parser(name)("just an answer, no call")
    assert plain.tool_calls == [] and plain.content == "just an answer, no call"


def test_tool_parsers_keep_leading_text():
    from vllm_metax_b200.entrypoints.parsers import get_tool_parser

    assert get_tool_parser("internlm")('Let me check.<|action_start|><|plugin|>{"name": "f", "parameters": {}}<|action_end|>').content == "Let me check."
    assert get_tool_parser("qwen3_coder")("Sure.\n<tool_call>\n<function=f>\n</function>\n</tool_call>").content == "Sure."
    assert get_tool_parser("kimi_k2")('x<|tool_calls_section_begin|><|tool_call_begin|>functions.f:1<|tool_call_argument_begin|>{}'
                                      '<|tool_call_end|><|tool_calls_section_end|>').tool_calls[0].id == "functions.f:1"


def test_more_reasoning_formats():
    from vllm_metax_b200.entrypoints.parsers import get_reasoning_parser

    assert get_reasoning_parser("mistral")("[THINK]step 1[/THINK]42") == ("step 1", "42")
    assert get_reasoning_parser("granite")("Here is my thought process: a then b. Here is my response: yes") == ("a then b.", "yes")
    assert get_reasoning_parser("granite")("plain") == (None, "plain")
    assert get_reasoning_parser("hunyuan_a13b")("<think>hm</think>\n<answer>\nyes\n</answer>") == ("hm", "yes")
