"""Cascade (shared-prefix) attention: requests whose leading cache blocks are the same physical blocks attend that
prefix in one pass per step; tokens must equal the engine that reads the prefix once per request."""
import os

import torch

from vllm_metax_b200 import LLM, SamplingParams
from tests.test_e2e_plumbing import tiny_cfg


def _generate(cascade: bool, prompts, shared):
    os.environ["B200_CASCADE_ATTENTION"] = "1" if cascade else "0"
    os.environ["B200_CASCADE_MIN_SAVED_TOKENS"] = "64"
    try:
        llm = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64,
                  num_gpu_blocks=96, enable_prefix_caching=True)
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        llm.generate([shared + [7]], SamplingParams(max_tokens=1, ignore_eos=True))        # fills the prefix cache
        outs = llm.generate(prompts, sp)
        return llm, [o.outputs[0].token_ids for o in outs], [o.num_cached_tokens for o in outs]
    finally:
        os.environ.pop("B200_CASCADE_ATTENTION", None)
        os.environ.pop("B200_CASCADE_MIN_SAVED_TOKENS", None)


def test_cascade_matches_per_request_attention():
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, 1024, (80,), generator=g).tolist()            # five full blocks of 16
    prompts = [shared + torch.randint(0, 1024, (n,), generator=g).tolist() for n in (5, 40, 1, 19, 70)]
    plain_llm, want, cached = _generate(False, prompts, shared)
    casc_llm, got, cached2 = _generate(True, prompts, shared)
    assert cached == cached2 == [80] * 5                                    # all five start from the shared blocks
    assert got == want
    assert getattr(casc_llm.engine.runner, "cascade_steps", 0) > 0
    assert getattr(plain_llm.engine.runner, "cascade_steps", 0) == 0


import pytest  # noqa: E402


@pytest.mark.gpu
def test_cascade_on_gpu_close_to_per_request_attention(kernel_status_ok):
    """Same comparison on the device kernels (bf16: the merged result rounds differently, so first tokens must agree
    and the continuations mostly)."""
    from vllm_metax_b200 import ModelConfig

    cfg = dict(architecture="LlamaForCausalLM", vocab_size=2048, hidden_size=1024, intermediate_size=2816,
               num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
               max_position_embeddings=1024, dtype=torch.bfloat16, seed=0)
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, 2048, (256,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 1, 19, 70, 33)]
    res = {}
    for cascade in (False, True):
        os.environ["B200_CASCADE_ATTENTION"] = "1" if cascade else "0"
        os.environ["B200_CASCADE_MIN_SAVED_TOKENS"] = "64"
        try:
            llm = LLM(ModelConfig(**cfg), device="cuda", block_size=64, max_model_len=512, max_num_seqs=8,
                      max_num_batched_tokens=256, num_gpu_blocks=64, enable_prefix_caching=True)
            llm.generate([shared + [7]], SamplingParams(max_tokens=1, ignore_eos=True))
            outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
            res[cascade] = ([list(o.outputs[0].token_ids) for o in outs], getattr(llm.engine.runner, "cascade_steps", 0))
            llm.engine.runner.graphs.clear()
            del llm
            torch.cuda.empty_cache()
        finally:
            os.environ.pop("B200_CASCADE_ATTENTION", None)
            os.environ.pop("B200_CASCADE_MIN_SAVED_TOKENS", None)
    (want, n0), (got, n1) = res[False], res[True]
    assert n0 == 0 and n1 > 0
    assert [t[0] for t in got] == [t[0] for t in want], (got, want)
    prefix = [next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), len(y)) for x, y in zip(got, want)]
    assert min(prefix) >= 2 and sum(prefix) >= 3 * len(want), (prefix, got, want)
