"""Regex- and JSON-schema-guided decoding with a character-level toy tokenizer: whatever the (random) model prefers,
the decoded output must match the pattern."""
import json
import os
import sys

import pytest
import regex
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)
CHARS = [chr(c) for c in range(32, 127)]


class CharTokenizer:
    """Token i < 95 is one printable ASCII character; a few multi-character tokens follow; the rest decode to ''."""
    chat_template = None
    multi = ['{"', '":', '", "', "true", "false", "null", "12", '"}', "ab"]

    def piece(self, t):
        if t < len(CHARS):
            return CHARS[t]
        if t - len(CHARS) < len(self.multi):
            return self.multi[t - len(CHARS)]
        return ""

    def encode(self, text, add_special_tokens=True):
        return [CHARS.index(c) for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(self.piece(int(t)) for t in ids)


def test_schema_to_regex_subset():
    from vllm_metax_b200.engine.structured import schema_to_regex

    rx = schema_to_regex({"type": "object", "properties": {
        "name": {"type": "string"}, "age": {"type": "integer"}, "ok": {"type": "boolean"},
        "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 2}}})
    good = ['{"name": "x y", "age": 3, "ok": true, "tags": ["a", "b"]}', '{"name":"","age":-12,"ok":false,"tags":[]}']
    bad = ['{"name": 1, "age": 3, "ok": true, "tags": []}', '{"name":"x","age":3,"ok":true,"tags":["a","b","a"]}',
           '{"age":3,"name":"x","ok":true,"tags":[]}']
    assert all(regex.fullmatch(rx, g) for g in good) and not any(regex.fullmatch(rx, b) for b in bad)
    assert all(json.loads(g) for g in good)
    with pytest.raises(NotImplementedError):
        schema_to_regex({"anyOf": []})


@pytest.fixture(scope="module")
def llm():
    from vllm_metax_b200 import LLM

    return LLM(tiny_cfg(), tokenizer=CharTokenizer(), **KW)


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_guided_regex(llm, temperature):
    from vllm_metax_b200 import SamplingParams

    pattern = r"(yes|no), [0-9]{3}-[a-c]+!"
    sp = SamplingParams(max_tokens=40, temperature=temperature, seed=1, guided_regex=pattern)
    outs = llm.generate(["Q: ok?", "Q: sure?", "x"], sp)
    for o in outs:
        assert regex.fullmatch(pattern, o.outputs[0].text), o.outputs[0].text
        assert o.outputs[0].finish_reason == "stop"


def test_guided_json(llm):
    from vllm_metax_b200 import SamplingParams

    schema = {"type": "object", "properties": {"city": {"enum": ["Paris", "Rome"]}, "n": {"enum": [1, 22, 333]},
                                               "ok": {"type": "boolean"}}}
    outs = llm.generate(["a", "bb"], SamplingParams(max_tokens=60, guided_json=schema))
    for o in outs:
        doc = json.loads(o.outputs[0].text)
        assert set(doc) == {"city", "n", "ok"} and doc["city"] in ("Paris", "Rome") and doc["n"] in (1, 22, 333)
    # unbounded parts (an integer of any length): a run cut off by max_tokens is still a prefix of a valid document
    from vllm_metax_b200.engine.structured import schema_to_regex

    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "s": {"type": "string"}}}
    o = llm.generate(["c"], SamplingParams(max_tokens=30, guided_json=schema))[0].outputs[0]
    assert regex.fullmatch(schema_to_regex(schema), o.text, partial=True), o.text
    # the multi-character tokens are usable too (the guide works on decoded text, not on single characters)
    from vllm_metax_b200.engine.structured import RegexGuide

    g = RegexGuide(r'\{"k":true\}', CharTokenizer())
    row = torch.zeros(1024)
    row[95] = 5.0                                    # token '{"' has the best logit and is a valid start
    assert g.allowed([], row, None)[0] == 95


def test_guided_needs_tokenizer():
    from vllm_metax_b200 import LLM, SamplingParams

    with pytest.raises(ValueError):
        LLM(tiny_cfg(), **KW).generate([[1, 2]], SamplingParams(guided_regex="a+"))


def test_schema_to_regex_optional_refs_alternatives():
    """``required`` decides which properties may be left out; ``$ref`` / ``anyOf`` / type lists / formats expand."""
    import regex

    from vllm_metax_b200.engine.structured import schema_to_regex

    def ok(schema, doc):
        return regex.fullmatch(schema_to_regex(schema), doc) is not None

    s = {"type": "object", "required": ["b"],
         "properties": {"a": {"type": "integer"}, "b": {"type": "string"}, "c": {"type": "boolean"}}}
    assert ok(s, '{"b": "x"}') and ok(s, '{"a": 1, "b": "x"}') and ok(s, '{"a": 1, "b": "x", "c": true}')
    assert ok(s, '{"b": "x", "c": false}')
    assert not ok(s, '{"a": 1}') and not ok(s, '{"a": 1, "c": true}') and not ok(s, '{"b": "x",}')
    none_required = dict(s, required=[])
    assert ok(none_required, "{}") and ok(none_required, '{"c": true}') and ok(none_required, '{"a": 1, "c": true}')
    assert not ok(none_required, '{"c": true, "a": 1}')                       # listed order is kept
    people = {"$defs": {"P": {"type": "object", "properties": {
        "name": {"type": "string"}, "age": {"anyOf": [{"type": "integer"}, {"type": "null"}]}}}},
        "type": "array", "items": {"$ref": "#/$defs/P"}, "minItems": 1}
    assert ok(people, '[{"name": "a", "age": null}, {"name": "b", "age": 3}]') and not ok(people, "[]")
    misc = {"type": "object", "properties": {"id": {"type": "string", "format": "uuid"},
                                             "t": {"type": ["string", "null"], "maxLength": 3},
                                             "tags": {"type": "array", "items": {}}}}
    assert ok(misc, '{"id": "123e4567-e89b-12d3-a456-426614174000", "t": "abc", "tags": [1, "x", {"k": 2}]}')
    assert ok(misc, '{"id": "123e4567-e89b-12d3-a456-426614174000", "t": null, "tags": []}')
    assert not ok(misc, '{"id": "123e4567-e89b-12d3-a456-426614174000", "t": "abcd", "tags": []}')
    assert ok({"type": "string", "pattern": "^[a-z]+\\d$"}, '"abc1"') and not ok({"type": "string", "pattern": "^[a-z]+\\d$"}, '"abc"')
    assert ok({}, '{"a": [1, 2], "b": {"c": null}}')
    tree = {"$defs": {"N": {"type": "object", "properties": {"v": {"type": "integer"},
                                                                "kids": {"type": "array", "items": {"$ref": "#/$defs/N"}}},
                            "required": ["v"]}}, "$ref": "#/$defs/N"}
    # a recursive definition is one named group that calls itself: exact at any depth
    assert ok(tree, '{"v": 1, "kids": [{"v": 2, "kids": [{"v": 3, "kids": [{"v": 4, "kids": [{"v": 5}]}]}]}, {"v": 6}]}')
    assert not ok(tree, '{"v": 1, "kids": [{"v": 2, "kids": [{"v": "x"}]}]}')
    assert regex.fullmatch(schema_to_regex(tree), '{"v": 1, "kids": [{"v": 2, "ki', partial=True)
    import pytest as _pytest
    with _pytest.raises(NotImplementedError):
        schema_to_regex({"$defs": {"A": {"$ref": "#/$defs/A"}}, "$ref": "#/$defs/A"})


@pytest.mark.parametrize("lo,hi", [(0, 9), (1, 100), (17, 342), (95, 1003), (-20, 15), (-250, -13), (0, 0), (7, 7),
                                   (1000, 99999), (None, 42), (5, None), (-3, None), (None, -11)])
def test_integer_range_regex_is_exact(lo, hi):
    from vllm_metax_b200.engine.structured import integer_range_regex

    rx = regex.compile(integer_range_regex(lo, hi))
    a = (lo if lo is not None else -1500) - 30
    b = (hi if hi is not None else 1500) + 30
    for v in list(range(a, b + 1)) + [10 ** 6, -10 ** 6, 123456]:
        want = (lo is None or v >= lo) and (hi is None or v <= hi)
        assert bool(rx.fullmatch(str(v))) == want, (lo, hi, v)
    assert not rx.fullmatch("007") and not rx.fullmatch("-0") and not rx.fullmatch("1.0")


def test_schema_ranges_and_all_of():
    from vllm_metax_b200.engine.structured import schema_to_regex

    rx = schema_to_regex({"type": "object", "properties": {"age": {"type": "integer", "minimum": 1, "maximum": 120},
                                                          "n": {"type": "integer", "exclusiveMinimum": 0}}})
    assert regex.fullmatch(rx, '{"age": 120, "n": 1}') and regex.fullmatch(rx, '{"age": 1, "n": 99999}')
    assert not regex.fullmatch(rx, '{"age": 121, "n": 1}') and not regex.fullmatch(rx, '{"age": 5, "n": 0}')
    merged = schema_to_regex({"$defs": {"base": {"type": "object", "properties": {"id": {"type": "integer"}}, "required": ["id"]}},
                              "allOf": [{"$ref": "#/$defs/base"},
                                        {"properties": {"name": {"type": "string"}}, "required": ["name"]}]})
    assert regex.fullmatch(merged, '{"id": 3, "name": "x"}') and not regex.fullmatch(merged, '{"id": 3}')
    with pytest.raises(NotImplementedError):
        schema_to_regex({"allOf": [{"properties": {"a": {"type": "string"}}}, {"properties": {"a": {"type": "integer"}}}]})


def test_open_values_nest_to_any_depth():
    """A schema that leaves a value open (``{}``, an object without properties, an array without ``items``) accepts
    JSON of any nesting depth through one recursive definition; partial matching follows it too."""
    from vllm_metax_b200.engine.structured import schema_to_regex

    rx = regex.compile(schema_to_regex({"type": "object"}))
    deep = '{"a": {"b": [1, "x", null, {"q": [[[{"r": {"s": []}}]]]}]}, "c": true}'
    assert rx.fullmatch(deep)
    assert not rx.fullmatch("[1]") and not rx.fullmatch('{"a"}') and not rx.fullmatch('{"a": [1,]}')
    m = rx.fullmatch(deep[:40], partial=True)
    assert m is not None and m.partial
    assert rx.fullmatch('{"a": 1}}', partial=True) is None
    mixed = regex.compile(schema_to_regex({"type": "object", "properties": {"k": {"type": "string"}, "meta": {},
                                                                           "tags": {"type": "array"}}}))
    assert mixed.fullmatch('{"k": "v", "meta": {"x": [1, {"y": null}]}, "tags": [[1], "a"]}')
    assert not mixed.fullmatch('{"k": 3, "meta": 1, "tags": []}')
    closed = schema_to_regex({"type": "object", "properties": {"k": {"type": "string"}}})
    assert "(?(DEFINE)" not in closed                       # nothing open: no definition in front


_SQL = r'''
# a tiny query language
root   ::= "SELECT " column (", " column){0,2} " FROM " table (" WHERE " cond)? ";"
column ::= "name" | "age" | "id"
table  ::= [a-z_]{1,8}
cond   ::= column " " op " " value
op     ::= "=" | "<" | ">" | "<="
value  ::= [0-9]{1,3} | "'" [^'\n]{0,6} "'"
'''

_ARITH = r'''
root ::= expr
expr ::= term (ws [-+] ws term)*
term ::= factor (ws [*/] ws factor)*
factor ::= number | "(" ws expr ws ")"
number ::= "-"? [0-9]+ ("." [0-9]+)?
ws ::= " "*
'''


def test_grammar_to_pattern():
    from vllm_metax_b200.engine.grammar import grammar_to_regex

    sql = regex.compile(grammar_to_regex(_SQL))
    assert sql.fullmatch("SELECT name FROM users;") and sql.fullmatch("SELECT name, age FROM t WHERE id <= 120;")
    assert sql.fullmatch("SELECT id FROM t WHERE name = 'bob #';")          # '#' inside a class or string is no comment
    assert not sql.fullmatch("SELECT foo FROM t;") and not sql.fullmatch("SELECT name FROM t WHERE id = 1234;")
    assert sql.fullmatch("SELECT name, a", partial=True) and sql.fullmatch("SELECT x", partial=True) is None
    arith = regex.compile(grammar_to_regex(_ARITH))                         # nesting: a context-free language
    assert arith.fullmatch("1 + 2 * (3 - 4.5)") and arith.fullmatch("((((1))))")
    assert not arith.fullmatch("(1 + ") and arith.fullmatch("(1 + ", partial=True)
    assert arith.fullmatch("1 + + 2", partial=True) is None and arith.fullmatch("(1 + 2))", partial=True) is None
    esc = regex.compile(grammar_to_regex('root ::= "a\\"b\\n" [\\]x-z]+ "\\x41\\u00e9" other-rule\nother-rule ::= .'))
    assert esc.fullmatch('a"b\n]zy' + "Aé" + "\n") and not esc.fullmatch('a"b\n]w' + "Aé!")
    with pytest.raises(NotImplementedError, match="left-recursive"):
        grammar_to_regex('root ::= expr\nexpr ::= expr "+" [0-9] | [0-9]')
    with pytest.raises(NotImplementedError, match="left-recursive"):     # hidden behind a rule that can be empty
        grammar_to_regex('root ::= ws root "x" | "y"\nws ::= " "*')
    for bad in ('root ::= foo', 'x ::= "a"', 'root ::= "a" )', 'root ::= "a', 'root ::= [a-z', 'root ::= "a"{3,1}',
                'root ::= "a"\nroot ::= "b"', 'nothing here'):
        with pytest.raises(ValueError):
            grammar_to_regex(bad)


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_guided_grammar(llm, temperature):
    from vllm_metax_b200 import SamplingParams
    from vllm_metax_b200.engine.grammar import grammar_to_regex

    sp = SamplingParams(max_tokens=80, temperature=temperature, seed=3, guided_grammar=_SQL)
    rx = regex.compile(grammar_to_regex(_SQL))
    for o in llm.generate(["q1", "another"], sp):
        out = o.outputs[0]
        assert rx.fullmatch(out.text, partial=True), out.text
        assert out.finish_reason == "stop" and rx.fullmatch(out.text), out.text    # every repetition is bounded: it must end
    o = llm.generate(["calc"], SamplingParams(max_tokens=24, temperature=temperature, seed=5, guided_grammar=_ARITH))[0].outputs[0]
    assert regex.fullmatch(grammar_to_regex(_ARITH), o.text, partial=True), o.text
    with pytest.raises(ValueError):
        llm.generate(["x"], SamplingParams(guided_grammar=_SQL, guided_regex="a+"))
