"""Constrained decoding: a choice, a regular expression, a JSON schema.

    python examples/structured_outputs.py --model /path/to/hf_model
"""
import argparse

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    a = ap.parse_args()
    llm = LLM(a.model)
    cases = [
        ("Is the sky blue? Answer:", SamplingParams(max_tokens=4, guided_choice=[" yes", " no"])),
        ("A US phone number:", SamplingParams(max_tokens=20, guided_regex=r" \(\d{3}\) \d{3}-\d{4}")),
        ("Describe Paris as JSON:", SamplingParams(max_tokens=80, guided_json={
            "type": "object", "properties": {"city": {"type": "string"}, "population": {"type": "integer"},
                                           "capital": {"type": "boolean"}}})),
    ]
    for prompt, sp in cases:
        print(repr(prompt), "->", repr(llm.generate([prompt], sp)[0].outputs[0].text))


if __name__ == "__main__":
    main()
