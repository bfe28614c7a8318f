"""Disaggregated prefill through the shared-storage connector: a producer engine publishes prompt KV, a consumer
engine loads it instead of recomputing; missing / corrupt blocks fall back to recomputation with identical output
(reference pattern: examples/disaggregated/kv_load_failure_recovery_offline)."""
import glob
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)


def _cfg(path, role):
    return {"kv_connector": "SharedStorageConnector", "kv_role": role,
            "kv_connector_extra_config": {"shared_storage_path": path}}


def test_chain_hashes_are_prefix_stable():
    from vllm_metax_b200.kv_transfer.shared_storage import chain_hashes

    a = chain_hashes(list(range(40)), 16)
    b = chain_hashes(list(range(33)) + [7] * 20, 16)
    assert len(a) == 2 and a == b[:2] and len(b) == 3
    assert chain_hashes(list(range(40)), 16, salt=("lora", 1)) != a


def test_prefill_decode_split_and_failure_recovery(tmp_path):
    from vllm_metax_b200 import LLM, SamplingParams

    store = str(tmp_path / "kv")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (100, 37, 16)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM(tiny_cfg(), **KW).generate(prompts, sp)]

    producer = LLM(tiny_cfg(), kv_transfer_config=_cfg(store, "kv_producer"), **KW)
    producer.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
    assert producer.engine.kv_connector.stats["blocks_saved"] == 100 // 16 + 37 // 16 + 16 // 16
    assert len(glob.glob(os.path.join(store, "*.kv"))) == 9

    consumer = LLM(tiny_cfg(), kv_transfer_config=_cfg(store, "kv_consumer"), **KW)
    outs = consumer.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    # prompt of 100: 6 blocks (96 tokens); 37: 2 blocks; 16: (16 - 1) // 16 = 0 blocks (one token must be computed)
    assert consumer.engine.stats["kv_external_tokens"] == 96 + 32
    assert consumer.engine.stats["prefill_tokens"] == (100 - 96) + (37 - 32) + 16
    assert [o.num_cached_tokens for o in outs] == [96, 32, 0]

    # corrupt one block of the longest prompt and delete another: the valid prefix is kept, the rest recomputed
    from vllm_metax_b200.kv_transfer.shared_storage import chain_hashes

    hs = chain_hashes(prompts[0], 16)
    with open(os.path.join(store, hs[3] + ".kv"), "r+b") as f:
        f.seek(100)
        f.write(b"\xff\xff\xff\xff")
    os.remove(os.path.join(store, chain_hashes(prompts[1], 16)[0] + ".kv"))
    again = LLM(tiny_cfg(), kv_transfer_config=_cfg(store, "kv_consumer"), **KW)
    outs = again.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    assert [o.num_cached_tokens for o in outs] == [48, 0, 0]
    assert again.engine.stats["kv_load_failures"] == 1 and again.engine.kv_connector.stats["load_failures"] == 1
    assert again.engine.kv.num_free_blocks == 64                       # nothing leaked on the failure path
