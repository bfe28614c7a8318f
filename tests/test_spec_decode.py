"""Speculative decoding: n-gram proposer, the verification rule, and end-to-end equality with plain decoding."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200.engine.spec_decode import NgramProposer, SpeculativeConfig, verify


def test_ngram_proposer():
    p = NgramProposer(SpeculativeConfig(num_speculative_tokens=3, prompt_lookup_max=3))
    assert p.propose([1, 2, 3, 4, 9, 1, 2, 3]) == [4, 9, 1]
    assert p.propose([5, 6, 7]) == []
    assert p.propose([1, 2, 1, 2, 1]) == [2, 1]          # most recent earlier match of the longest tail


def test_verify_rule():
    assert verify([5, 6, 7], [5, 6, 9, 1]) == [5, 6, 9]
    assert verify([5, 6, 7], [5, 6, 7, 8]) == [5, 6, 7, 8]
    assert verify([5], [4, 0]) == [4]
    assert verify([], [3]) == [3]


def _cfg():
    return ModelConfig(architecture="LlamaForCausalLM", vocab_size=32, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       max_position_embeddings=512, dtype=torch.float32)


@pytest.mark.parametrize("k", [1, 4])
def test_spec_decode_matches_plain_greedy_cpu(k):
    # a tiny vocabulary makes the random model repeat itself, so the n-gram proposer gets real acceptances
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256, seed=0)
    prompts = [[1, 2, 3, 1, 2, 3, 1, 2], [7, 7, 7, 7], [3, 9, 4, 3, 9, 4, 3]]
    sp = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
    plain = LLM(_cfg(), **kw).generate(prompts, sp)
    spec_llm = LLM(_cfg(), speculative_config={"method": "ngram", "num_speculative_tokens": k}, **kw)
    spec = spec_llm.generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    st = spec_llm.engine.stats
    assert st["draft_tokens"] > 0 and st["accepted_tokens"] > 0
    assert st["steps"] < 3 * 40          # fewer engine steps than tokens generated


def test_spec_decode_respects_max_tokens_and_stop_cpu():
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=64, block_size=16, max_model_len=256, seed=0)
    llm = LLM(_cfg(), speculative_config={"method": "ngram", "num_speculative_tokens": 4}, **kw)
    out = llm.generate([[1, 2, 3, 1, 2, 3, 1, 2]], SamplingParams(max_tokens=7, temperature=0.0, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 7
    ref = LLM(_cfg(), **kw).generate([[1, 2, 3, 1, 2, 3, 1, 2]], SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True))
    stop_tok = ref[0].outputs[0].token_ids[5]
    out = llm.generate([[1, 2, 3, 1, 2, 3, 1, 2]], SamplingParams(max_tokens=30, temperature=0.0, stop_token_ids=[stop_tok]))
    toks = out[0].outputs[0].token_ids
    assert toks[-1] == stop_tok and stop_tok not in toks[:-1]


def _ds_cfg():
    return ModelConfig(architecture="DeepseekV3ForCausalLM", vocab_size=64, hidden_size=128, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, q_lora_rank=64,
                       kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_experts=4,
                       num_experts_per_tok=2, moe_intermediate_size=64, n_shared_experts=1, first_k_dense_replace=1,
                       n_group=2, topk_group=1, scoring_func="sigmoid", routed_scaling_factor=2.5,
                       num_nextn_predict_layers=1, max_position_embeddings=256, dtype=torch.float32)


def test_mtp_module_shapes_and_weight_names_cpu():
    from vllm_metax_b200.models import get_model_class

    cls = get_model_class("DeepSeekMTPModel")
    m = cls(_ds_cfg())
    names = dict(m.named_parameters())
    for n in ("model.layers.2.enorm.weight", "model.layers.2.hnorm.weight", "model.layers.2.eh_proj.weight",
              "model.layers.2.shared_head.norm.weight", "model.layers.2.shared_head.head.weight",
              "model.embed_tokens.weight", "model.layers.2.self_attn.o_proj.weight"):
        assert n in names, n
    # checkpoint-style names: the per-layer embedding copy lands on the shared embedding, target layers are ignored
    emb = torch.randn_like(names["model.embed_tokens.weight"])
    loaded = m.load_weights([("model.layers.2.embed_tokens.weight", emb),
                             ("model.layers.0.input_layernorm.weight", torch.ones(128)),
                             ("model.layers.2.enorm.weight", torch.full((128,), 2.0))])
    assert "model.embed_tokens.weight" in loaded and "model.layers.2.enorm.weight" in loaded
    assert torch.equal(names["model.embed_tokens.weight"].data, emb)


def test_mtp_spec_decode_matches_plain_greedy_cpu():
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=32, block_size=64, max_model_len=128, seed=0)
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7]]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    plain = LLM(_ds_cfg(), **kw).generate(prompts, sp)
    llm = LLM(_ds_cfg(), speculative_config={"method": "mtp", "num_speculative_tokens": 1}, **kw)
    spec = llm.generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert llm.engine.scheduler.num_draft_tokens > 0


def test_eagle_spec_decode_matches_plain_greedy_cpu():
    """An EAGLE head (random here, so few drafts are accepted) must never change the greedy output; drafts are
    proposed every step and the head shares the target's embedding and language-model head."""
    from tests.test_e2e_plumbing import tiny_cfg

    kw = dict(device="cpu", num_gpu_blocks=64, block_size=16, max_model_len=128, max_num_batched_tokens=32)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (5, 40, 17)]      # 40 > 32: chunked prefill
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    plain = LLM(tiny_cfg(), **kw).generate(prompts, sp)
    llm = LLM(tiny_cfg(), speculative_config={"method": "eagle", "num_speculative_tokens": 1}, **kw)
    head = llm.engine.proposer.module
    assert type(head).__name__ == "EagleLlamaForCausalLM" and head.fc.weight.shape == (256, 512)
    assert head.embed_tokens is llm.engine.runner.model.model.embed_tokens and head.lm_head is llm.engine.runner.model.lm_head
    spec = llm.generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert llm.engine.scheduler.num_draft_tokens > 0
    # published EAGLE checkpoints name their tensors fc.* / layers.0.* (with or without a model. prefix)
    names = {"fc.weight": torch.zeros(256, 512), "fc.bias": torch.zeros(256),
             "model.layers.0.self_attn.q_proj.weight": torch.zeros(256, 256),
             "layers.0.mlp.down_proj.weight": torch.zeros(256, 512)}
    assert head.load_weights(names.items()) == {"fc.weight", "fc.bias", "layers.0.self_attn.qkv_proj.weight",
                                                "layers.0.mlp.down_proj.weight"}
