"""Pipeline parallel and decode context parallel (one process per GPU).

    torchrun --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 examples/pipeline_and_context_parallel.py \
        --model /path/to/hf_model --tp 2 --pp 2
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/pipeline_and_context_parallel.py \
        --model /path/to/mqa_model --tp 2 --dcp 2          # KV heads replicated over the 2 ranks

Every rank runs the same script; rank 0 prints.
"""
import argparse
import os

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dcp", type=int, default=1)
    a = ap.parse_args()
    llm = LLM(a.model, tensor_parallel_size=a.tp, pipeline_parallel_size=a.pp, decode_context_parallel_size=a.dcp)
    outs = llm.generate(["The three laws of robotics are", "A haiku about NVLink:"], SamplingParams(max_tokens=48))
    if int(os.environ.get("RANK", "0")) == 0:
        for o in outs:
            print(repr(o.outputs[0].text))


if __name__ == "__main__":
    main()
