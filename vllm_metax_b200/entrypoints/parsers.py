"""Tool-call and reasoning parsers for the chat endpoint.

A served model writes tool calls and its chain of thought as plain text in a model-specific markup; the OpenAI
response separates them into ``message.tool_calls`` / ``message.reasoning_content`` / ``message.content``.  Each parser
here turns the finished text (or the text so far, for streaming) into those parts.

Tool-call formats:
  hermes       ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Hermes, Qwen2.5 / Qwen3)
  llama3_json  a bare JSON object (or several, ``;``-separated) ``{"name": ..., "parameters": {...}}``, optionally
               after ``<|python_tag|>``
  mistral      ``[TOOL_CALLS] [{"name": ..., "arguments": {...}}, ...]``
  deepseek_v3  ``<｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>``
  pythonic     ``[get_weather(city="Paris"), other(x=1)]``
  deepseek_v31 ``<｜tool▁call▁begin｜>NAME<｜tool▁sep｜>{...}<｜tool▁call▁end｜>``
  granite / granite-20b-fc / phi4_mini_json / minimax / hunyuan_a13b / jamba / internlm / xlam
               a JSON list (or objects) of calls after the model's marker (``<|tool_call|>``, ``<function_call>``,
               ``functools``, ``<tool_calls>...</tool_calls>``, ``<|action_start|><|plugin|>``, a bare / fenced list)
  kimi_k2      ``<|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{...}<|tool_call_end|>``
  qwen3_coder  ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter></function></tool_call>``
  glm45        ``<tool_call>NAME <arg_key>K</arg_key><arg_value>V</arg_value></tool_call>``
Reasoning formats:
  deepseek_r1 / qwen3   ``<think> ... </think>`` before the answer (the opening tag may be part of the prompt)

The reference serves through upstream's OpenAI server, whose ``--tool-call-parser`` / ``--reasoning-parser`` options
these mirror (examples/online_serving/openai_chat_completion_client_with_tools.py and
openai_chat_completion_with_reasoning.py in the reference tree use them).
"""
from __future__ import annotations

import ast
import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Callable, Optional


@dataclass
class ToolCall:
    name: str
    arguments: str                        # JSON text, as the OpenAI schema wants it
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: Optional[int] = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ParsedMessage:
    content: Optional[str]
    tool_calls: list = field(default_factory=list)
    reasoning_content: Optional[str] = None


def _args_text(args) -> str:
    if isinstance(args, str):
        try:
            json.loads(args)
            return args
        except ValueError:
            return json.dumps(args)
    return json.dumps(args if args is not None else {}, ensure_ascii=False)


def _call_from_obj(obj) -> Optional[ToolCall]:
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    return ToolCall(obj["name"], _args_text(args))


def _json_objects(text: str) -> list:
    """Every top-level JSON value that can be decoded from ``text``, scanning left to right."""
    dec = json.JSONDecoder()
    out, i = [], 0
    while i < len(text):
        if text[i] in "{[":
            try:
                val, end = dec.raw_decode(text, i)
                out.append((i, end, val))
                i = end
                continue
            except ValueError:
                pass
        i += 1
    return out


# ----------------------------------------------------------------------------------------------- tool parsers
def parse_hermes(text: str) -> ParsedMessage:
    calls, rest, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", text, flags=re.S):
        try:
            c = _call_from_obj(json.loads(m.group(1)))
        except ValueError:
            c = None
        if c is None:
            continue
        calls.append(c)
        rest.append(text[pos:m.start()])
        pos = m.end()
    rest.append(text[pos:])
    content = "".join(rest).strip()
    return ParsedMessage(content or None, calls) if calls else ParsedMessage(text)


def parse_llama3_json(text: str) -> ParsedMessage:
    body = text.split("<|python_tag|>", 1)[1] if "<|python_tag|>" in text else text
    stripped = body.strip()
    if not stripped.startswith("{"):
        return ParsedMessage(text)
    calls = []
    for part in stripped.split(";"):
        objs = _json_objects(part)
        if len(objs) != 1 or part[:objs[0][0]].strip() or part[objs[0][1]:].strip():
            return ParsedMessage(text)
        c = _call_from_obj(objs[0][2])
        if c is None:
            return ParsedMessage(text)
        calls.append(c)
    return ParsedMessage(None, calls) if calls else ParsedMessage(text)


def parse_mistral(text: str) -> ParsedMessage:
    if "[TOOL_CALLS]" not in text:
        return ParsedMessage(text)
    head, tail = text.split("[TOOL_CALLS]", 1)
    calls = []
    for _, _, val in _json_objects(tail):
        for obj in (val if isinstance(val, list) else [val]):
            c = _call_from_obj(obj)
            if c is not None:
                calls.append(c)
    return ParsedMessage(head.strip() or None, calls) if calls else ParsedMessage(text)


_DS_CALL = re.compile(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>(?P<name>[^\n]+)\n```json\n(?P<args>.*?)\n```"
                      r"\s*<｜tool▁call▁end｜>", re.S)


def parse_deepseek_v3(text: str) -> ParsedMessage:
    calls = [ToolCall(m.group("name").strip(), _args_text(m.group("args").strip())) for m in _DS_CALL.finditer(text)]
    if not calls:
        return ParsedMessage(text)
    head = text.split("<｜tool▁calls▁begin｜>", 1)[0] if "<｜tool▁calls▁begin｜>" in text else _DS_CALL.split(text)[0]
    return ParsedMessage(head.strip() or None, calls)


def parse_pythonic(text: str) -> ParsedMessage:
    s = text.strip()
    if not (s.startswith("[") and s.endswith("]")):
        return ParsedMessage(text)
    try:
        tree = ast.parse(s, mode="eval").body
    except SyntaxError:
        return ParsedMessage(text)
    if not isinstance(tree, ast.List) or not tree.elts:
        return ParsedMessage(text)
    calls = []
    for node in tree.elts:
        if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and not node.args):
            return ParsedMessage(text)
        try:
            args = {kw.arg: ast.literal_eval(kw.value) for kw in node.keywords}
        except (ValueError, SyntaxError):
            return ParsedMessage(text)
        calls.append(ToolCall(node.func.id, json.dumps(args, ensure_ascii=False)))
    return ParsedMessage(None, calls)


def _calls_from_json_list(blob: str) -> list:
    """Tool calls from text that holds a JSON list (or consecutive JSON objects) of ``{"name", "arguments" | "parameters"}``."""
    calls = []
    for _, _, val in _json_objects(blob):
        for obj in (val if isinstance(val, list) else [val]):
            c = _call_from_obj(obj)
            if c is not None:
                calls.append(c)
    return calls


def _tagged_json_parser(open_tag: str, close_tag: Optional[str]):
    """Formats that put a JSON list / objects of calls after ``open_tag`` (up to ``close_tag`` when there is one)."""
    def parse(text: str) -> ParsedMessage:
        if open_tag not in text:
            return ParsedMessage(text)
        head, tail = text.split(open_tag, 1)
        if close_tag and close_tag in tail:
            tail = tail.split(close_tag, 1)[0]
        calls = _calls_from_json_list(tail)
        return ParsedMessage(head.strip() or None, calls) if calls else ParsedMessage(text)
    return parse


parse_granite = _tagged_json_parser("<|tool_call|>", None)                       # <|tool_call|>[{...}, ...]
parse_granite_20b_fc = _tagged_json_parser("<function_call>", None)              # <function_call> {...}
parse_phi4_mini_json = _tagged_json_parser("functools", None)                    # functools[{...}, ...]
parse_minimax = _tagged_json_parser("<tool_calls>", "</tool_calls>")             # one JSON object per line
parse_hunyuan_a13b = _tagged_json_parser("<tool_calls>", "</tool_calls>")        # a JSON list
parse_jamba = _tagged_json_parser("<tool_calls>", "</tool_calls>")


def parse_internlm(text: str) -> ParsedMessage:
    """``...<|action_start|><|plugin|>{"name": ..., "parameters": {...}}<|action_end|>``"""
    m = re.search(r"<\|action_start\|>\s*<\|plugin\|>(.*?)(?:<\|action_end\|>|$)", text, flags=re.S)
    if not m:
        return ParsedMessage(text)
    calls = _calls_from_json_list(m.group(1))
    return ParsedMessage(text[:m.start()].strip() or None, calls) if calls else ParsedMessage(text)


def parse_xlam(text: str) -> ParsedMessage:
    """A JSON list of calls, bare, inside a ```json fence, after ``</think>`` or after ``[TOOL_CALLS]``."""
    body = text.split("</think>", 1)[1] if "</think>" in text else text
    body = body.split("[TOOL_CALLS]", 1)[1] if "[TOOL_CALLS]" in body else body
    fence = re.search(r"```(?:json)?\s*(.*?)```", body, flags=re.S)
    blob = (fence.group(1) if fence else body).strip()
    if not blob.startswith("["):
        return ParsedMessage(text)
    calls = _calls_from_json_list(blob)
    lead = body[:fence.start()].strip() if fence else None
    return ParsedMessage(lead or None, calls) if calls else ParsedMessage(text)


_KIMI_CALL = re.compile(r"<\|tool_call_begin\|>\s*(?P<id>[^<\s]+)\s*<\|tool_call_argument_begin\|>\s*(?P<args>.*?)\s*"
                        r"<\|tool_call_end\|>", re.S)


def parse_kimi_k2(text: str) -> ParsedMessage:
    """``<|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{...}
    <|tool_call_end|><|tool_calls_section_end|>``"""
    calls = []
    for m in _KIMI_CALL.finditer(text):
        ident = m.group("id")
        name = ident.split(":", 1)[0]
        name = name.split(".", 1)[1] if name.startswith("functions.") else name
        calls.append(ToolCall(name, _args_text(m.group("args")), id=ident))
    if not calls:
        return ParsedMessage(text)
    return ParsedMessage(text.split("<|tool_calls_section_begin|>", 1)[0].strip() or None, calls)


_DS31_CALL = re.compile(r"<｜tool▁call▁begin｜>(?P<name>.*?)<｜tool▁sep｜>(?P<args>.*?)<｜tool▁call▁end｜>", re.S)


def parse_deepseek_v31(text: str) -> ParsedMessage:
    """``<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>NAME<｜tool▁sep｜>{...}<｜tool▁call▁end｜><｜tool▁calls▁end｜>``"""
    calls = [ToolCall(m.group("name").strip(), _args_text(m.group("args").strip())) for m in _DS31_CALL.finditer(text)]
    if not calls:
        return ParsedMessage(text)
    return ParsedMessage(text.split("<｜tool▁calls▁begin｜>", 1)[0].strip() or None, calls)


def _typed(value: str):
    """Parameter text of the XML-style formats: JSON where it parses (numbers, booleans, objects), else the string."""
    v = value.strip("\n")
    try:
        return json.loads(v)
    except ValueError:
        return v


def parse_qwen3_coder(text: str) -> ParsedMessage:
    """``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``"""
    calls = []
    for fm in re.finditer(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", text, flags=re.S):
        args = {pm.group(1): _typed(pm.group(2))
                for pm in re.finditer(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", fm.group(2), flags=re.S)}
        calls.append(ToolCall(fm.group(1), json.dumps(args, ensure_ascii=False)))
    if not calls:
        return ParsedMessage(text)
    head = re.split(r"<tool_call>|<function=", text, maxsplit=1)[0]
    return ParsedMessage(head.strip() or None, calls)


def parse_glm45(text: str) -> ParsedMessage:
    """``<tool_call>NAME\n<arg_key>K</arg_key>\n<arg_value>V</arg_value>...</tool_call>``"""
    calls = []
    for m in re.finditer(r"<tool_call>\s*([^\n<]+)\s*(.*?)\s*(?:</tool_call>|$)", text, flags=re.S):
        keys = re.findall(r"<arg_key>(.*?)</arg_key>", m.group(2), flags=re.S)
        vals = re.findall(r"<arg_value>(.*?)</arg_value>", m.group(2), flags=re.S)
        calls.append(ToolCall(m.group(1).strip(), json.dumps({k.strip(): _typed(v) for k, v in zip(keys, vals)},
                                                             ensure_ascii=False)))
    if not calls:
        return ParsedMessage(text)
    return ParsedMessage(text.split("<tool_call>", 1)[0].strip() or None, calls)


TOOL_PARSERS: dict[str, Callable[[str], ParsedMessage]] = {
    "hermes": parse_hermes, "qwen": parse_hermes, "llama3_json": parse_llama3_json, "llama4_json": parse_llama3_json,
    "mistral": parse_mistral, "deepseek_v3": parse_deepseek_v3, "pythonic": parse_pythonic,
    "llama4_pythonic": parse_pythonic, "deepseek_v31": parse_deepseek_v31, "granite": parse_granite,
    "granite-20b-fc": parse_granite_20b_fc, "internlm": parse_internlm, "phi4_mini_json": parse_phi4_mini_json,
    "minimax": parse_minimax, "hunyuan_a13b": parse_hunyuan_a13b, "jamba": parse_jamba, "xlam": parse_xlam,
    "kimi_k2": parse_kimi_k2, "qwen3_coder": parse_qwen3_coder, "qwen3_xml": parse_qwen3_coder, "glm45": parse_glm45,
}


# ----------------------------------------------------------------------------------------------- reasoning parsers
def split_think(text: str, open_tag: str = "<think>", close_tag: str = "</think>", finished: bool = True):
    """``(reasoning, answer)``.  The opening tag is optional (chat templates of R1-style models end the prompt with
    it); without a closing tag everything so far is reasoning - unless the text is finished and never opened one."""
    body = text
    opened = False
    if open_tag in body:
        body = body.split(open_tag, 1)[1]
        opened = True
    if close_tag in body:
        reasoning, answer = body.split(close_tag, 1)
        return reasoning.strip() or None, answer.lstrip("\n") or None
    if opened or not finished:
        return body.strip() or None, None
    return None, text


def split_mistral_think(text: str, finished: bool = True):
    """Magistral: ``[THINK] ... [/THINK]answer``."""
    return split_think(text, "[THINK]", "[/THINK]", finished)


def split_granite(text: str, finished: bool = True):
    """Granite 3.2: ``Here is my thought process: ... Here is my response: ...`` (either phrase may start with
    "Here's")."""
    m = re.search(r"Here(?: is|'s) my thought process:(.*?)(?:Here(?: is|'s) my response:(.*))?$", text, flags=re.S)
    if not m:
        return None, text
    return (m.group(1).strip() or None), ((m.group(2) or "").strip() or None)


def split_hunyuan(text: str, finished: bool = True):
    """Hunyuan-A13B: ``<think>...</think><answer>...</answer>``."""
    reasoning, answer = split_think(text, finished=finished)
    if answer:
        m = re.search(r"<answer>\s*(.*?)\s*(?:</answer>|$)", answer, flags=re.S)
        answer = m.group(1) if m else answer
    return reasoning, answer or None


REASONING_PARSERS: dict[str, Callable] = {
    "deepseek_r1": split_think, "qwen3": split_think, "glm45": split_think, "step3": split_think,
    "mistral": split_mistral_think, "granite": split_granite, "hunyuan_a13b": split_hunyuan,
}


def get_tool_parser(name: Optional[str]):
    if not name:
        return None
    if name not in TOOL_PARSERS:
        raise ValueError(f"unknown tool-call parser {name!r} (known: {sorted(TOOL_PARSERS)})")
    return TOOL_PARSERS[name]


def get_reasoning_parser(name: Optional[str]):
    if not name:
        return None
    if name not in REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {name!r} (known: {sorted(REASONING_PARSERS)})")
    return REASONING_PARSERS[name]


def parse_chat_output(text: str, tool_parser=None, reasoning_parser=None, tools_requested: bool = False,
                      forced_tool: Optional[str] = None) -> ParsedMessage:
    """Reasoning first, then tool calls in what remains.  ``forced_tool``: ``tool_choice`` named one function and the
    output was constrained to its arguments - the whole answer is that call.  ``forced_tool=True``:
    ``tool_choice="required"``, the output was constrained to a JSON list ``[{"name": ..., "parameters": {...}}, ...]``
    (a list cut off by the token limit is answered as plain content)."""
    reasoning = None
    if reasoning_parser is not None:
        reasoning, text = reasoning_parser(text)
        text = text or ""
    if forced_tool is True:
        try:
            calls = json.loads(text)
            return ParsedMessage(None, [ToolCall(c["name"], json.dumps(c.get("parameters", {}))) for c in calls], reasoning)
        except (ValueError, KeyError, TypeError):
            return ParsedMessage(text or None, [], reasoning)
    if forced_tool:
        return ParsedMessage(None, [ToolCall(forced_tool, _args_text(text.strip() or "{}"))], reasoning)
    msg = tool_parser(text) if (tool_parser is not None and tools_requested) else ParsedMessage(text or None)
    msg.reasoning_content = reasoning
    return msg
