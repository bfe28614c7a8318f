"""Decode context parallel through the engine on CPU ranks (gloo): TP2 x DCP2 with one (replicated) KV head - every
rank keeps every second token of each sequence; greedy tokens must equal the single-process run, across chunked
prefill (context pass + merge), batched decode and prefix-cache hits."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402
from tests.test_tp_cpu import export_hf_checkpoint  # noqa: E402


def _worker(rank, world, port, path, prompts, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=world, decode_context_parallel_size=world, block_size=8,
                  max_model_len=256, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks=64, dtype=torch.float32,
                  enable_prefix_caching=True)
        assert llm.engine.runner.dcp == 2 and llm.engine.kv.block_size == 16       # 8 local slots x 2 ranks per block
        sp = SamplingParams(max_tokens=8, ignore_eos=True)
        first = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        second = [o.outputs[0].token_ids for o in llm.generate(prompts[:2], sp)]         # prefix-cache hits
        q.put((rank, first, second))
    except BaseException as e:
        q.put((rank, repr(e), None))
        raise


def test_dcp2_matches_single_process(tmp_path):
    from vllm_metax_b200 import LLM, SamplingParams

    kw = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks=64)
    ref_llm = LLM(tiny_cfg(num_key_value_heads=1), **kw)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (21, 77, 1, 40)]   # 77 > one chunk of 32
    want = [o.outputs[0].token_ids for o in ref_llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    path = str(tmp_path / "ckpt")
    export_hf_checkpoint(ref_llm.engine.runner.model, path)
    import json
    cfg = json.load(open(os.path.join(path, "config.json")))
    cfg["num_key_value_heads"] = 1
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + (os.getpid() % 150)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, path, prompts, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, first, second in got:
        assert first == want, (rank, first)
        assert second == want[:2], (rank, second)


def _mla_worker(rank, world, port, path, prompts, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=world, decode_context_parallel_size=world, block_size=8,
                  max_model_len=256, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks=64, dtype=torch.float32)
        assert llm.engine.runner.dcp == 2 and llm.engine.runner.dcp_per_token
        toks = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        q.put((rank, toks))
    except BaseException as e:
        q.put((rank, repr(e)))
        raise


def test_dcp2_mla_matches_single_process(tmp_path):
    """DeepSeek-V3 (MLA) with TP2 x DCP2 on CPU ranks: the latent cache is interleaved over the two ranks; chunked
    prefill (77 tokens > one 32-token chunk), mixed steps and batched decode give the single-process tokens."""
    tf = pytest.importorskip("transformers")
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    cfg = tf.DeepseekV3Config(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                              max_position_embeddings=256, intermediate_size=256, moe_intermediate_size=64,
                              n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, n_group=2, topk_group=1,
                              first_k_dense_replace=1, q_lora_rank=48, kv_lora_rank=512, qk_nope_head_dim=32,
                              qk_rope_head_dim=64, v_head_dim=32, num_key_value_heads=4)
    path = str(tmp_path / "ckpt")
    tf.DeepseekV3ForCausalLM(cfg).save_pretrained(path)
    kw = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=4, max_num_batched_tokens=32,
              num_gpu_blocks=64, dtype=torch.float32)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 77, 1, 40)]
    want = [o.outputs[0].token_ids for o in LLM(path, **kw).generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 150)
    procs = [ctx.Process(target=_mla_worker, args=(r, 2, port, path, prompts, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, toks in got:
        assert toks == want, (rank, toks, want)
