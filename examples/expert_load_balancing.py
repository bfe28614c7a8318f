"""Expert-parallel load balancing (EPLB) on a tensor- / expert-parallel MoE engine.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/expert_load_balancing.py <model dir>

``num_redundant_experts`` extra expert slots are spread over the ranks; every ``eplb_step_interval`` engine steps the
routing statistics of the last ``eplb_window`` steps are summed over the ranks, hot experts get more copies, the copies
are packed evenly, and the expert weights move between the ranks in place.  Generated tokens do not depend on it.
(The reference's use case: examples/offline_inference/data_parallel.py with --enable-eplb and
examples/ray_serving/elastic_ep of the reference tree.)
"""
import os
import sys

from vllm_metax_b200 import LLM, SamplingParams

model = sys.argv[1] if len(sys.argv) > 1 else "Qwen/Qwen3-30B-A3B"
world = int(os.environ.get("WORLD_SIZE", "1"))
llm = LLM(model, tensor_parallel_size=world, enable_expert_parallel=True, enable_eplb=True,
          num_redundant_experts=2 * world, eplb_step_interval=200, eplb_window=100)
prompts = ["The capital of France is", "Mixture-of-experts models route every token to"] * 32
outs = llm.generate(prompts, SamplingParams(max_tokens=256, temperature=0.0))
if int(os.environ.get("RANK", "0")) == 0:
    st = llm.engine.stats
    print(outs[0].outputs[0].text)
    print("re-placements:", st.get("eplb_rearrangements", 0), "balancedness (mean / max pairs per rank):",
          st.get("eplb_balancedness_before"), "->", st.get("eplb_balancedness_after"))
