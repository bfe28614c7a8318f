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


def test_network_connector_serves_blocks_over_tcp():
    """Producer and consumer engines joined by the TCP connector (loopback): the consumer pulls the prompt blocks
    from the producer's memory; a damaged blob and a vanished producer both end in recomputation, same tokens."""
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.kv_transfer.shared_storage import chain_hashes

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (100, 37, 16)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM(tiny_cfg(), **KW).generate(prompts, sp)]

    producer = LLM(tiny_cfg(), kv_transfer_config={"kv_connector": "NetworkKVConnector", "kv_role": "kv_producer",
                                                   "kv_connector_extra_config": {"listen": "127.0.0.1:0"}}, **KW)
    pc = producer.engine.kv_connector
    producer.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
    assert pc.stats["blocks_saved"] == 9 and pc.address.startswith("127.0.0.1:")

    def consumer():
        return LLM(tiny_cfg(), kv_transfer_config={"kv_connector": "NetworkKVConnector", "kv_role": "kv_consumer",
                                                   "kv_connector_extra_config": {"peers": [pc.address], "timeout_s": 2}}, **KW)

    c = consumer()
    outs = c.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    assert [o.num_cached_tokens for o in outs] == [96, 32, 0]
    assert c.engine.kv_connector.stats["blocks_loaded"] == 8 and c.engine.kv_connector.stats["bytes_received"] > 0
    c.engine.kv_connector.close()

    # a blob damaged in the producer's store fails its checksum on the consumer: prefix kept, rest recomputed
    h = chain_hashes(prompts[0], 16)[3]
    blob = bytearray(pc.store.blobs[h])
    blob[100:104] = b"\xff\xff\xff\xff"
    pc.store.blobs[h] = bytes(blob)
    c = consumer()
    outs = c.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want
    assert [o.num_cached_tokens for o in outs] == [48, 32, 0] and c.engine.stats["kv_load_failures"] == 1
    c.engine.kv_connector.close()

    # the producer goes away: lookups find nothing, everything is computed locally
    pc.close()
    c = consumer()
    outs = c.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in outs] == want and [o.num_cached_tokens for o in outs] == [0, 0, 0]


def test_block_store_is_bounded_lru():
    from vllm_metax_b200.kv_transfer.network import BlockStore

    st = BlockStore(max_bytes=250)
    for i in range(4):
        st.put(f"h{i}", bytes(100))
    assert not st.has("h0") and not st.has("h1") and st.has("h2") and st.has("h3") and st.size == 200
    st.get("h2")
    st.put("h4", bytes(100))
    assert st.has("h2") and not st.has("h3")


def test_host_offload_tier_in_one_engine():
    """kv_both on the host-memory connector: a prompt seen before is attached from host memory (the device-side
    prefix cache is off), shared prefixes hit, tokens do not change, and a bounded store evicts the oldest blocks."""
    from vllm_metax_b200 import LLM, SamplingParams

    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, 1024, (80,), generator=g).tolist()
    prompts = [base, base[:48] + torch.randint(0, 1024, (20,), generator=g).tolist()]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM(tiny_cfg(), **KW).generate(prompts, sp)]
    cfg = {"kv_connector": "OffloadingConnector", "kv_role": "kv_both",
           "kv_connector_extra_config": {"cpu_bytes_to_use": 1 << 30}}
    llm = LLM(tiny_cfg(), kv_transfer_config=cfg, **KW)
    first = llm.generate([prompts[0]], sp)
    assert first[0].outputs[0].token_ids == want[0] and first[0].num_cached_tokens == 0
    assert llm.engine.kv_connector.stats["blocks_saved"] == 80 // 16
    outs = llm.generate(prompts, sp)                              # the same prompt again, and one sharing 48 tokens
    assert [o.outputs[0].token_ids for o in outs] == want
    assert [o.num_cached_tokens for o in outs] == [64, 48]        # (80 - 1) // 16 * 16 and the shared 3 blocks
    assert llm.engine.stats["kv_external_tokens"] == 64 + 48
    # a store that holds about two blocks: old blocks fall out, loads stop at the first gap, tokens stay right
    blob = len(llm.engine.kv_connector._pack(0))
    small = LLM(tiny_cfg(), kv_transfer_config=dict(cfg, kv_connector_extra_config={"cpu_bytes_to_use": 2 * blob + 8}), **KW)
    small.generate([prompts[0]], sp)
    assert len(small.engine.kv_connector.store.blobs) == 2
    again = small.generate([prompts[0]], sp)[0]
    assert again.outputs[0].token_ids == want[0] and again.num_cached_tokens == 0      # the first block is gone
