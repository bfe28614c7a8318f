"""Data-parallel replicas behind one front (one GPU per replica by default).

    python examples/data_parallel.py --model /path/to/hf_model --dp 4
"""
import argparse

from vllm_metax_b200 import SamplingParams
from vllm_metax_b200.engine.dp import DataParallelLLM


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--dp", type=int, default=2)
    a = ap.parse_args()
    llm = DataParallelLLM(a.model, data_parallel_size=a.dp)
    prompts = [f"Question {i}: what is {i} squared?" for i in range(64)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=32))
    print("replica of each prompt:", llm.last_assignment)
    print(outs[0].outputs[0].text)
    llm.shutdown()


if __name__ == "__main__":
    main()
