"""Several LoRA adapters in one engine, chosen per request.

    python examples/multilora_inference.py --model /path/to/hf_model --lora sql=/path/to/peft_a --lora chat=/path/to/peft_b
"""
import argparse

from vllm_metax_b200 import LLM, SamplingParams
from vllm_metax_b200.lora import LoRARequest


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--lora", action="append", default=[], help="name=path of a PEFT adapter directory (repeatable)")
    ap.add_argument("--prompt", default="Write a SQL query that lists all users.")
    a = ap.parse_args()
    llm = LLM(a.model, enable_lora=True, max_loras=max(1, len(a.lora)), max_lora_rank=64)
    reqs = [None] + [LoRARequest(n, i + 1, p) for i, (n, p) in enumerate(s.split("=", 1) for s in a.lora)]
    outs = llm.generate([a.prompt] * len(reqs), SamplingParams(max_tokens=64), lora_request=reqs)
    for r, o in zip(reqs, outs):
        print(f"[{r.lora_name if r else 'base'}] {o.outputs[0].text}")


if __name__ == "__main__":
    main()
