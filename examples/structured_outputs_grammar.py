"""Grammar-guided and JSON-mode decoding.

    python examples/structured_outputs_grammar.py MODEL_DIR

* ``guided_grammar``: a context-free grammar in GBNF / EBNF notation; the output is a sentence of it.
* ``guided_json={"type": "object"}``: any JSON object, nested to any depth (what ``response_format: json_object``
  of the HTTP server maps to).
* a recursive JSON schema (a tree): exact, not unrolled.
"""
import sys

from vllm_metax_b200 import LLM, SamplingParams

SQL = r'''
root   ::= "SELECT " column (", " column)* " FROM " table (" WHERE " cond)? ";"
column ::= "name" | "age" | "id"
table  ::= [a-z_]+
cond   ::= column " " ("=" | "<" | ">") " " [0-9]{1,3}
'''

TREE = {"$defs": {"node": {"type": "object", "required": ["label"],
                           "properties": {"label": {"type": "string", "maxLength": 12},
                                          "children": {"type": "array", "maxItems": 3, "items": {"$ref": "#/$defs/node"}}}}},
        "$ref": "#/$defs/node"}


def main() -> None:
    llm = LLM(sys.argv[1], max_model_len=2048)
    runs = [("Write a SQL query that lists the names of the people older than 30.\n", SamplingParams(max_tokens=64, guided_grammar=SQL)),
            ("Describe Paris as a JSON object.\n", SamplingParams(max_tokens=128, guided_json={"type": "object"})),
            ("A small taxonomy of animals as a JSON tree.\n", SamplingParams(max_tokens=160, guided_json=TREE))]
    for prompt, sp in runs:
        out = llm.generate([prompt], sp)[0].outputs[0]
        print(f"{prompt.strip()!r}\n  -> {out.text!r} ({out.finish_reason})")


if __name__ == "__main__":
    main()
