"""Disaggregated prefill with a damaged KV store: the consumer recomputes what it cannot load.

    python examples/kv_load_failure_recovery.py --model /path/to/hf_model

A producer engine publishes the KV blocks of a prompt to a shared directory; one block file is then truncated.  The
consumer engine finds the prompt in the store, loads the intact leading blocks, notices the bad one (length / checksum
mismatch), releases the blocks from there on and prefills the rest itself, so the answer is the same as without the
store; ``engine.stats`` counts the failure and the tokens that did come from the store.
"""
import argparse
import glob
import os
import tempfile

from vllm_metax_b200 import LLM, SamplingParams


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    a = ap.parse_args()
    store = tempfile.mkdtemp(prefix="kv_store_")
    cfg = lambda role: {"kv_connector": "SharedStorageConnector", "kv_role": role,        # noqa: E731
                        "kv_connector_extra_config": {"shared_storage_path": store}}
    sp = SamplingParams(max_tokens=24, temperature=0.0)
    prompt = "Summarise the history of the transistor in three sentences. " * 12
    producer = LLM(a.model, kv_transfer_config=cfg("kv_producer"), max_model_len=2048)
    want = producer.generate([prompt], sp)[0].outputs[0].text
    files = sorted(glob.glob(os.path.join(store, "**", "*"), recursive=True))
    files = [f for f in files if os.path.isfile(f)]
    victim = files[len(files) // 2]
    with open(victim, "r+b") as f:
        f.truncate(max(1, os.path.getsize(victim) // 2))
    print(f"published {len(files)} block files, truncated {os.path.basename(victim)}")
    del producer
    consumer = LLM(a.model, kv_transfer_config=cfg("kv_consumer"), max_model_len=2048)
    got = consumer.generate([prompt], sp)[0].outputs[0].text
    st = consumer.engine.stats
    print("load failures:", st.get("kv_load_failures", 0), " tokens taken from the store:", st.get("kv_external_tokens", 0))
    print("same answer as the producer:", got == want)


if __name__ == "__main__":
    main()
