"""Prefill on one engine, decode on another, KV handed over through a shared directory.

    python examples/disaggregated_prefill.py --model /path/to/hf_model --store /dev/shm/b200_kv

In production the two engines are two server processes (``b200-serve --kv-transfer-config '{...}'``) on different
GPUs; here they run one after the other in one process to show the data flow.
"""
import argparse

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--store", default="/dev/shm/b200_kv")
    a = ap.parse_args()
    prompts = ["The capital of France is", "Blackwell tensor cores accumulate in"]

    def cfg(role):
        return {"kv_connector": "SharedStorageConnector", "kv_role": role,
                "kv_connector_extra_config": {"shared_storage_path": a.store}}

    prefill = LLM(a.model, kv_transfer_config=cfg("kv_producer"), gpu_memory_utilization=0.4)
    prefill.generate(prompts, SamplingParams(max_tokens=1))
    print("published blocks:", prefill.engine.kv_connector.stats["blocks_saved"])
    decode = LLM(a.model, kv_transfer_config=cfg("kv_consumer"), gpu_memory_utilization=0.4)
    for o in decode.generate(prompts, SamplingParams(max_tokens=32)):
        print(f"{o.prompt!r} -> {o.outputs[0].text!r} (prompt tokens taken from the store: {o.num_cached_tokens})")
    print("load failures (recomputed):", decode.engine.stats.get("kv_load_failures", 0))


if __name__ == "__main__":
    main()
