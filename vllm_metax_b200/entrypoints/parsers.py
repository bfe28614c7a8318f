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


TOOL_PARSERS: dict[str, Callable[[str], ParsedMessage]] = {
    "hermes": parse_hermes, "qwen": parse_hermes, "llama3_json": parse_llama3_json, "llama4_json": parse_llama3_json,
    "mistral": parse_mistral, "deepseek_v3": parse_deepseek_v3, "pythonic": parse_pythonic,
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


REASONING_PARSERS: dict[str, Callable] = {
    "deepseek_r1": split_think, "qwen3": split_think, "glm45": split_think, "step3": split_think,
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
    output was constrained to its arguments - the whole answer is that call."""
    reasoning = None
    if reasoning_parser is not None:
        reasoning, text = reasoning_parser(text)
        text = text or ""
    if forced_tool:
        return ParsedMessage(None, [ToolCall(forced_tool, _args_text(text.strip() or "{}"))], reasoning)
    msg = tool_parser(text) if (tool_parser is not None and tools_requested) else ParsedMessage(text or None)
    msg.reasoning_content = reasoning
    return msg
