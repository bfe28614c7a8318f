"""Weight hand-over from a trainer to the serving engine, as RLHF loops do between optimisation steps.

    python examples/rlhf_weight_sync.py --model /path/to/hf_model

The engine goes to sleep (KV cache and, at level 2, weights leave the device) while the "trainer" owns the GPU, wakes
up, receives the new tensors under their checkpoint names through ``update_weights`` (fused and sharded parameters are
rebuilt by the same loaders a checkpoint goes through) and generates with them.
"""
import argparse

import torch

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    a = ap.parse_args()
    llm = LLM(a.model, enable_sleep_mode=True, max_model_len=512)
    sp = SamplingParams(max_tokens=16, temperature=0.0)
    prompt = "The three primary colours are"
    print("before:", repr(llm.generate([prompt], sp)[0].outputs[0].text))

    llm.sleep(level=1)                    # the trainer's turn on the device
    # ... a policy-gradient step would run here; this stands in for its result: a nudged final norm
    new = {"model.norm.weight": llm.engine.runner.model.state_dict()["model.norm.weight"].float().mul(1.02).cpu()}
    llm.wake_up()
    n = llm.update_weights(new.items())
    print(f"updated {n} tensor(s)")
    print("after: ", repr(llm.generate([prompt], sp)[0].outputs[0].text))
    # every rank of a tensor-parallel engine runs this same script; collective_rpc names a model-runner method
    print("kv bytes per block:", llm.collective_rpc("kv_bytes_per_block"))


if __name__ == "__main__":
    main()
