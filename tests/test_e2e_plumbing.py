"""CPU plumbing run: tiny Llama through the whole engine (scheduler, paged KV cache with
block_size 16, chunked prefill, greedy sampling) against a plain PyTorch forward."""
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams


def tiny_cfg(**kw):
    d = dict(architecture="LlamaForCausalLM", vocab_size=1024, hidden_size=256, intermediate_size=512,
             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5,
             rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32, seed=0)
    d.update(kw)
    return ModelConfig(**d)


def plain_forward(model, ids):
    """Dense (no cache, no paging) causal forward of the same weights; returns logits [L, V]."""
    cfg = model.cfg
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    L = len(ids)
    x = model.model.embed_tokens.weight[torch.tensor(ids)].float()
    pos = torch.arange(L)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))
    fr = torch.outer(pos.float(), inv)
    cos, sin = fr.cos()[:, None, :], fr.sin()[:, None, :]

    def rope(t):
        t1, t2 = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

    def norm(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w.float()

    for i in range(cfg.num_hidden_layers):
        lyr = model.model.layers[str(i)]
        h = norm(x, lyr.input_layernorm.weight)
        qkv = h @ lyr.self_attn.qkv_proj.weight.float().t()
        q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
        q, k, v = rope(q.view(L, H, D)), rope(k.view(L, Hkv, D)), v.view(L, Hkv, D)
        k, v = k.repeat_interleave(H // Hkv, 1), v.repeat_interleave(H // Hkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * D ** -0.5
        s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1)[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(L, H * D)
        x = x + a @ lyr.self_attn.o_proj.weight.float().t()
        h = norm(x, lyr.post_attention_layernorm.weight)
        gu = h @ lyr.mlp.gate_up_proj.weight.float().t()
        g, u = gu[:, 0::2], gu[:, 1::2]   # gate / up rows are stored interleaved
        x = x + (torch.nn.functional.silu(g) * u) @ lyr.mlp.down_proj.weight.float().t()
    x = norm(x, model.model.norm.weight)
    return x @ model.lm_head.weight.float().t()[:, : cfg.vocab_size]


def greedy_reference(model, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain_forward(model, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_plumbing_greedy_matches_plain_forward():
    llm = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=128, max_num_seqs=8,
              max_num_batched_tokens=64, num_gpu_blocks=64)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (32,), generator=g).tolist() for _ in range(4)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True))
    model = llm.engine.runner.model
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == greedy_reference(model, p, 16)
        assert o.finished and o.outputs[0].finish_reason == "length"
        assert o.metrics.ttft is not None and o.metrics.tpot is not None


def test_chunked_prefill_and_preemption_keep_results():
    """A token budget smaller than a prompt (chunking) and a KV pool too small for all requests
    (preemption + recompute) must not change greedy outputs."""
    cfg = tiny_cfg()
    big = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=256,
              num_gpu_blocks=64)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 17, 33, 5)]
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in big.generate(prompts, sp)]
    small = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=24,
                num_gpu_blocks=9)
    small.engine.runner.model.load_state_dict(big.engine.runner.model.state_dict())
    got = [o.outputs[0].token_ids for o in small.generate(prompts, sp)]
    assert got == want
    assert small.engine.stats["preemptions"] > 0


def test_prefix_caching_hits_and_matches():
    cfg = tiny_cfg()
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=128,
              num_gpu_blocks=64, enable_prefix_caching=True)
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, 1024, (48,), generator=g).tolist()
    p1, p2 = shared + [1, 2, 3], shared + [7, 8]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    o1 = llm.generate([p1], sp)[0]
    o2 = llm.generate([p2], sp)[0]
    assert o2.num_cached_tokens == 48
    model = llm.engine.runner.model
    assert o1.outputs[0].token_ids == greedy_reference(model, p1, 6)
    assert o2.outputs[0].token_ids == greedy_reference(model, p2, 6)
