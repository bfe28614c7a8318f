"""Architectures against their Hugging Face implementations (tiny random checkpoints, fp32, CPU): the checkpoint is
written by ``save_pretrained`` and read by this engine's loader, so name mapping, fused-qkv layouts, position schemes
(rotary fraction, ALiBi slope schedules, learned tables), residual wiring and activations are all covered.  Checked:
mean final hidden state over every prompt position (numeric) and greedy continuations (token-exact)."""
import pytest
import torch

tf = pytest.importorskip("transformers")

BASE = dict(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=256)
GPT = dict(vocab_size=512, n_embd=128, n_layer=2, n_head=4, n_positions=256)
CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2)),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2, head_dim=32)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2, sliding_window=None)),
    "neox": ("GPTNeoXConfig", "GPTNeoXForCausalLM", dict(BASE, intermediate_size=256)),
    "neox_sequential": ("GPTNeoXConfig", "GPTNeoXForCausalLM",
                        dict(BASE, intermediate_size=256, use_parallel_residual=False, rotary_pct=0.5)),
    "falcon_grouped": ("FalconConfig", "FalconForCausalLM", dict(BASE, new_decoder_architecture=True, num_kv_heads=2)),
    "falcon_multi_query": ("FalconConfig", "FalconForCausalLM", dict(BASE, multi_query=True, parallel_attn=True)),
    "falcon_rw_alibi": ("FalconConfig", "FalconForCausalLM",
                        dict(BASE, multi_query=False, parallel_attn=False, alibi=True, bias=True)),
    "bloom": ("BloomConfig", "BloomForCausalLM", dict(vocab_size=512, hidden_size=128, n_layer=2, n_head=4)),
    "bloom_6_heads": ("BloomConfig", "BloomForCausalLM", dict(vocab_size=512, hidden_size=192, n_layer=2, n_head=6)),
    "mpt": ("MptConfig", "MptForCausalLM", dict(vocab_size=512, d_model=128, n_layers=2, n_heads=4, max_seq_len=256)),
    "bigcode_multi_query": ("GPTBigCodeConfig", "GPTBigCodeForCausalLM", dict(GPT)),
    "bigcode_mha": ("GPTBigCodeConfig", "GPTBigCodeForCausalLM", dict(GPT, multi_query=False)),
    "gpt2": ("GPT2Config", "GPT2LMHeadModel", dict(GPT)),
}
PROMPTS = [[5, 9, 33, 100, 7, 8, 200, 31, 2, 17, 45, 301, 77, 12, 490, 3, 64, 65, 66, 9], [3, 4, 5, 6]]


@pytest.mark.parametrize("case", sorted(CASES))
def test_matches_hugging_face(case, tmp_path):
    from vllm_metax_b200 import LLM, SamplingParams

    cfg_cls, model_cls, kw = CASES[case]
    if not hasattr(tf, cfg_cls):
        pytest.skip(f"transformers has no {cfg_cls}")
    torch.manual_seed(0)
    hf = getattr(tf, model_cls)(getattr(tf, cfg_cls)(**kw)).eval().float()
    with torch.no_grad():
        for p in hf.parameters():          # default inits leave norms at 1 / biases at 0, and logits nearly flat
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=16, block_size=16)
    got_h = llm.embed(PROMPTS, pooling="mean", normalize=False)
    outs = llm.generate(PROMPTS, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    for i, ids in enumerate(PROMPTS):
        with torch.no_grad():
            t = torch.tensor([ids])
            want_h = hf.base_model(t).last_hidden_state[0].mean(0)
            want = hf.generate(t, max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        torch.testing.assert_close(got_h[i], want_h, atol=2e-4, rtol=2e-4)
        assert list(outs[i].outputs[0].token_ids) == want
