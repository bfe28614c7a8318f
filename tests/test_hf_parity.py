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
    "llama_all_bias": ("LlamaConfig", "LlamaForCausalLM",
                       dict(BASE, intermediate_size=256, num_key_value_heads=2, attention_bias=True, mlp_bias=True)),
    "ernie4_5": ("Ernie4_5Config", "Ernie4_5ForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2)),
    "glm": ("GlmConfig", "GlmForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2, head_dim=32, pad_token_id=0)),
    "glm4": ("Glm4Config", "Glm4ForCausalLM", dict(BASE, intermediate_size=256, num_key_value_heads=2, head_dim=32, pad_token_id=0)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                  dict(BASE, intermediate_size=256, moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2,
                       num_key_value_heads=2, head_dim=32, norm_topk_prob=True)),
    "qwen2_moe_shared_expert": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM",
                                dict(BASE, intermediate_size=256, moe_intermediate_size=64, shared_expert_intermediate_size=128,
                                     num_experts=8, num_experts_per_tok=2, num_key_value_heads=2)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM",
                dict(BASE, intermediate_size=128, num_local_experts=4, num_experts_per_tok=2, num_key_value_heads=2)),
    "deepseek_v2": ("DeepseekV2Config", "DeepseekV2ForCausalLM",
                    dict(BASE, intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8, num_experts_per_tok=2,
                         n_shared_experts=1, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=None,
                         kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32, num_key_value_heads=4)),
    "deepseek_v3": ("DeepseekV3Config", "DeepseekV3ForCausalLM",
                    dict(BASE, intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8, num_experts_per_tok=2,
                         n_shared_experts=1, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=48,
                         kv_lora_rank=512, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32, num_key_value_heads=4)),
    "glm4_moe": ("Glm4MoeConfig", "Glm4MoeForCausalLM",
                 dict(BASE, intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8, num_experts_per_tok=2,
                      n_shared_experts=1, n_group=2, topk_group=1, first_k_dense_replace=1, num_key_value_heads=2,
                      head_dim=32, use_qk_norm=True)),
    "ernie4_5_moe": ("Ernie4_5_MoeConfig", "Ernie4_5_MoeForCausalLM",
                     dict(BASE, intermediate_size=256, moe_intermediate_size=64, moe_num_experts=8, moe_k=2,
                          moe_num_shared_experts=1, moe_layer_start_index=1, num_key_value_heads=2)),
    "qwen3_next_hybrid": ("Qwen3NextConfig", "Qwen3NextForCausalLM",
                          dict(vocab_size=512, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                               head_dim=32, max_position_embeddings=256, intermediate_size=256, moe_intermediate_size=64,
                               shared_expert_intermediate_size=64, num_experts=8, num_experts_per_tok=2,
                               linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                               linear_value_head_dim=16, linear_conv_kernel_dim=4, norm_topk_prob=True)),
    "mamba": ("MambaConfig", "MambaForCausalLM",
              dict(vocab_size=512, hidden_size=64, state_size=8, num_hidden_layers=2, conv_kernel=4, expand=2,
                   time_step_rank=8, pad_token_id=0, bos_token_id=1, eos_token_id=2)),
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
            elif "moe" not in case and "mixtral" not in case and "deepseek" not in case and "qwen3_next" not in case:
                p.mul_(3.0)                # (routers stay at their init scale: near-ties flip experts in fp32)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):     # DeepSeek-V3 / GLM-4.5 routing bias: a buffer, zero at init
                b.add_(0.05 * torch.randn_like(b))
        for n, p in hf.named_parameters():
            if n.endswith("e_score_correction_bias"):     # Ernie keeps it as a [1, E] parameter
                p.copy_(0.02 * torch.randn_like(p))
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


# ------------------------------------------------------------------------------------------ checkpoint dialects
def _hf(model_cls, cfg_cls, **kw):
    torch.manual_seed(1)
    hf = getattr(tf, model_cls)(getattr(tf, cfg_cls)(**kw)).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.mul_(3.0)
    return hf


def _check(tmp_path, hf, tensors, config):
    import json

    from safetensors.torch import save_file

    from vllm_metax_b200 import LLM, SamplingParams

    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(dict(config, torch_dtype="float32")))
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


def _layer_items(sd, n_layers):
    for i in range(n_layers):
        pre = f"model.layers.{i}."
        yield i, {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}


def test_internlm2_dialect(tmp_path):
    """``wqkv`` holds, per kv head, its q heads followed by k and v; ``w1`` / ``w3`` / ``w2`` = gate / up / down."""
    H, Hkv, D, L = 4, 2, 32, 2
    hf = _hf("LlamaForCausalLM", "LlamaConfig", **dict(BASE, intermediate_size=256, num_key_value_heads=Hkv))
    sd = hf.state_dict()
    out = {"model.tok_embeddings.weight": sd["model.embed_tokens.weight"], "model.norm.weight": sd["model.norm.weight"],
           "output.weight": sd["lm_head.weight"]}
    for i, t in _layer_items(sd, L):
        q = t["self_attn.q_proj.weight"].reshape(Hkv, H // Hkv, D, -1)
        k = t["self_attn.k_proj.weight"].reshape(Hkv, 1, D, -1)
        v = t["self_attn.v_proj.weight"].reshape(Hkv, 1, D, -1)
        p = f"model.layers.{i}."
        out[p + "attention.wqkv.weight"] = torch.cat([q, k, v], 1).reshape((H + 2 * Hkv) * D, -1)
        out[p + "attention.wo.weight"] = t["self_attn.o_proj.weight"]
        out[p + "feed_forward.w1.weight"] = t["mlp.gate_proj.weight"]
        out[p + "feed_forward.w3.weight"] = t["mlp.up_proj.weight"]
        out[p + "feed_forward.w2.weight"] = t["mlp.down_proj.weight"]
        out[p + "attention_norm.weight"] = t["input_layernorm.weight"]
        out[p + "ffn_norm.weight"] = t["post_attention_layernorm.weight"]
    _check(tmp_path, hf, out, dict(BASE, architectures=["InternLM2ForCausalLM"], intermediate_size=256,
                                   num_key_value_heads=Hkv, rms_norm_eps=hf.config.rms_norm_eps, bias=False))


def test_baichuan_w_pack_dialect(tmp_path):
    hf = _hf("LlamaForCausalLM", "LlamaConfig", **dict(BASE, intermediate_size=256))
    sd = hf.state_dict()
    out = {k: v for k, v in sd.items() if "_proj" not in k or "mlp" in k or "o_proj" in k}
    for i, t in _layer_items(sd, 2):
        out[f"model.layers.{i}.self_attn.W_pack.weight"] = torch.cat(
            [t["self_attn.q_proj.weight"], t["self_attn.k_proj.weight"], t["self_attn.v_proj.weight"]], 0)
    _check(tmp_path, hf, out, dict(BASE, architectures=["BaichuanForCausalLM"], intermediate_size=256,
                                   rms_norm_eps=hf.config.rms_norm_eps))


def test_qwen1_dialect(tmp_path):
    """Qwen-1 names; ``w2`` is the gate, ``w1`` the up projection, ``intermediate_size`` counts both."""
    hf = _hf("Qwen2ForCausalLM", "Qwen2Config", **dict(BASE, intermediate_size=256, num_key_value_heads=4))
    sd = hf.state_dict()
    out = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.ln_f.weight": sd["model.norm.weight"],
           "lm_head.weight": sd["lm_head.weight"]}
    for i, t in _layer_items(sd, 2):
        p = f"transformer.h.{i}."
        for kind in ("weight", "bias"):
            out[p + f"attn.c_attn.{kind}"] = torch.cat([t[f"self_attn.{x}_proj.{kind}"] for x in "qkv"], 0)
        out[p + "attn.c_proj.weight"] = t["self_attn.o_proj.weight"]
        out[p + "mlp.w2.weight"] = t["mlp.gate_proj.weight"]
        out[p + "mlp.w1.weight"] = t["mlp.up_proj.weight"]
        out[p + "mlp.c_proj.weight"] = t["mlp.down_proj.weight"]
        out[p + "ln_1.weight"] = t["input_layernorm.weight"]
        out[p + "ln_2.weight"] = t["post_attention_layernorm.weight"]
    _check(tmp_path, hf, out, dict(architectures=["QWenLMHeadModel"], vocab_size=512, hidden_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, kv_channels=32, intermediate_size=512, seq_length=256,
                                   layer_norm_epsilon=hf.config.rms_norm_eps, rotary_emb_base=hf.config.rope_parameters["rope_theta"]))


def test_chatglm_dialect(tmp_path):
    """ChatGLM2/3 / GLM-4 original export: fused multi-query ``query_key_value`` (with bias), ``dense_h_to_4h`` = gate | up,
    half of every head rotated in adjacent pairs."""
    hf = _hf("GlmForCausalLM", "GlmConfig", **dict(BASE, intermediate_size=256, num_key_value_heads=2, head_dim=32, pad_token_id=0))
    sd = hf.state_dict()
    out = {"transformer.embedding.word_embeddings.weight": sd["model.embed_tokens.weight"],
           "transformer.encoder.final_layernorm.weight": sd["model.norm.weight"],
           "transformer.output_layer.weight": sd["lm_head.weight"],
           "transformer.rotary_pos_emb.inv_freq": torch.ones(8)}
    for i, t in _layer_items(sd, 2):
        p = f"transformer.encoder.layers.{i}."
        for kind in ("weight", "bias"):
            out[p + f"self_attention.query_key_value.{kind}"] = torch.cat([t[f"self_attn.{x}_proj.{kind}"] for x in "qkv"], 0)
        out[p + "self_attention.dense.weight"] = t["self_attn.o_proj.weight"]
        out[p + "mlp.dense_h_to_4h.weight"] = t["mlp.gate_up_proj.weight"]
        out[p + "mlp.dense_4h_to_h.weight"] = t["mlp.down_proj.weight"]
        out[p + "input_layernorm.weight"] = t["input_layernorm.weight"]
        out[p + "post_attention_layernorm.weight"] = t["post_attention_layernorm.weight"]
    _check(tmp_path, hf, out, dict(architectures=["ChatGLMModel"], padded_vocab_size=512, hidden_size=128, num_layers=2,
                                   num_attention_heads=4, kv_channels=32, ffn_hidden_size=256, seq_length=256,
                                   multi_query_attention=True, multi_query_group_num=2, add_qkv_bias=True, rmsnorm=True,
                                   layernorm_epsilon=hf.config.rms_norm_eps, rope_ratio=1.0))


def test_baichuan_13b_alibi(tmp_path):
    """ALiBi variant (hidden size != 4096 under the ``BaiChuanForCausalLM`` name) against a dense torch forward."""
    import json

    from safetensors.torch import save_file

    from vllm_metax_b200 import LLM
    from vllm_metax_b200.models.gpt import alibi_slopes

    H, D, L, hid = 4, 32, 2, 128
    hf = _hf("LlamaForCausalLM", "LlamaConfig", **dict(BASE, intermediate_size=256))
    sd = hf.state_dict()
    out = {k: v for k, v in sd.items() if "_proj" not in k or "mlp" in k or "o_proj" in k}
    for i, t in _layer_items(sd, L):
        out[f"model.layers.{i}.self_attn.W_pack.weight"] = torch.cat(
            [t["self_attn.q_proj.weight"], t["self_attn.k_proj.weight"], t["self_attn.v_proj.weight"]], 0)
    save_file({k: v.contiguous() for k, v in out.items()}, str(tmp_path / "model.safetensors"))
    eps = hf.config.rms_norm_eps
    (tmp_path / "config.json").write_text(json.dumps(dict(BASE, architectures=["BaiChuanForCausalLM"], intermediate_size=256,
                                                          rms_norm_eps=eps, torch_dtype="float32")))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=16, block_size=16)
    got = llm.embed([PROMPTS[0]], pooling="mean", normalize=False)[0]

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    ids = torch.tensor(PROMPTS[0])
    n = ids.numel()
    x = sd["model.embed_tokens.weight"][ids]
    pos = torch.arange(n)
    bias = alibi_slopes(H)[:, None, None] * (pos[None, None, :] - pos[None, :, None]).float()
    bias = bias.masked_fill(pos[None, None, :] > pos[None, :, None], float("-inf"))
    for i, t in _layer_items(sd, L):
        h = rms(x, t["input_layernorm.weight"])
        q, k, v = [(h @ t[f"self_attn.{c}_proj.weight"].T).reshape(n, H, D).transpose(0, 1) for c in "qkv"]
        a = torch.softmax(q @ k.transpose(1, 2) * D ** -0.5 + bias, -1) @ v
        x = x + a.transpose(0, 1).reshape(n, hid) @ t["self_attn.o_proj.weight"].T
        h = rms(x, t["post_attention_layernorm.weight"])
        x = x + (torch.nn.functional.silu(h @ t["mlp.gate_proj.weight"].T) * (h @ t["mlp.up_proj.weight"].T)) @ t["mlp.down_proj.weight"].T
    want = rms(x, sd["model.norm.weight"]).mean(0)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)


def test_qwen3_next_state_carry_across_chunks_and_batches(tmp_path):
    """The recurrent state and the convolution carry must survive chunked prefill (8 tokens per step here), batched
    decode with requests joining at different times, and slot reuse after a request finishes."""
    from vllm_metax_b200 import LLM, SamplingParams

    cfg_cls, model_cls, kw = CASES["qwen3_next_hybrid"]
    torch.manual_seed(2)
    hf = getattr(tf, model_cls)(getattr(tf, cfg_cls)(**kw)).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=32, block_size=16,
              max_num_batched_tokens=8, max_num_seqs=2, enable_prefix_caching=True)      # prefix caching is refused
    assert not llm.engine.kv.enable_prefix_caching
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 5, 27, 11)]  # 4 requests, 2 slots
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    for ids, o in zip(prompts, outs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                               pad_token_id=0)[0, len(ids):].tolist()
        assert list(o.outputs[0].token_ids) == want
    assert not llm.engine.runner.state_slots and len(llm.engine.runner.free_state_slots) == 2


def test_qwen3_next_recomputes_state_after_preemption(tmp_path):
    """With too few KV blocks for the batch a request is preempted and later re-computed from scratch; its recurrent
    state must restart from zero in a fresh slot."""
    from vllm_metax_b200 import LLM, SamplingParams

    cfg_cls, model_cls, kw = CASES["qwen3_next_hybrid"]
    torch.manual_seed(4)
    hf = getattr(tf, model_cls)(getattr(tf, cfg_cls)(**kw)).eval().float()
    hf.save_pretrained(str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", max_model_len=64, num_gpu_blocks=7, block_size=8,
              max_num_batched_tokens=32, max_num_seqs=3)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (14, 15, 13)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert llm.engine.scheduler.num_preemptions > 0
    for ids, o in zip(prompts, outs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([ids]), max_new_tokens=12, do_sample=False, eos_token_id=None,
                               pad_token_id=0)[0, len(ids):].tolist()
        assert list(o.outputs[0].token_ids) == want
    assert not llm.engine.runner.state_slots
