"""DeepSeek-V4 attention: the online compressor against the pooling written out, the attention layer (window +
compressed entries + sink + inverse RoPE + grouped output projection) against a per-token oracle across chunked,
batched steps, and the model end to end (chunk-size invariant tokens)."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200.attention.metadata import AttentionMetadata, ForwardContext, set_forward_context
from vllm_metax_b200.layers.v4_attention import (DeepseekV4Attention, V4Compressor, naive_compress, naive_v4_attention,
                                                 rope_tail)


def _cfg(**kw):
    base = dict(architecture="DeepseekV4ForCausalLM", vocab_size=64, hidden_size=64, intermediate_size=128,
                num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=2, head_dim=512, q_lora_rank=32,
                qk_rope_head_dim=64, o_lora_rank=16, o_groups=2, sliding_window=8, compress_ratios=[4, 128, 0],
                index_topk=4, index_n_heads=2, index_head_dim=128, num_experts=4, num_experts_per_tok=2,
                moe_intermediate_size=32, n_shared_experts=1, first_k_dense_replace=0, scoring_func="sqrtsoftplus",
                routed_scaling_factor=1.5, hc_mult=2, hc_sinkhorn_iters=5, num_hash_layers=1,
                max_position_embeddings=512, dtype=torch.float32)
    base.update(kw)
    return ModelConfig(**base)


def _steps(lengths, chunks):
    """Yields per step the list of (request, start, n)."""
    done = [0] * len(lengths)
    for sizes in chunks:
        parts = []
        for i, n in enumerate(sizes):
            n = min(n, lengths[i] - done[i])
            if n > 0:
                parts.append((i, done[i], n))
                done[i] += n
        if parts:
            yield parts
    assert done == list(lengths)


def _metadata(parts, blocks, bs):
    qsl, slots, pos = [0], [], []
    for i, s, n in parts:
        qsl.append(qsl[-1] + n)
        for p in range(s, s + n):
            pos.append(p)
            slots.append(blocks[i][p // bs] * bs + p % bs)
    bt = torch.zeros(len(parts), max(len(b) for b in blocks), dtype=torch.int32)
    for row, (i, _, _) in enumerate(parts):
        bt[row, : len(blocks[i])] = torch.tensor(blocks[i])
    md = AttentionMetadata(num_tokens=len(pos), num_reqs=len(parts), num_decodes=0, num_decode_tokens=0,
                           query_start_loc=torch.tensor(qsl, dtype=torch.int32),
                           seq_lens=torch.tensor([s + n for _, s, n in parts], dtype=torch.int32), block_table=bt,
                           slot_mapping=torch.tensor(slots), max_query_len=max(n for _, _, n in parts),
                           max_seq_len=max(s + n for _, s, n in parts), block_size=bs)
    md.extra["state_indices"] = torch.tensor([i for i, _, _ in parts], dtype=torch.int32)
    return md, torch.tensor(pos)


@pytest.mark.parametrize("ratio", [4, 128])
def test_online_compressor_matches_pooling(ratio):
    torch.manual_seed(0)
    cfg = _cfg()
    c = V4Compressor(cfg, 128, ratio, "c")
    torch.nn.init.normal_(c.fused_wkv_wgate.weight, std=0.3)
    c.ape.data.normal_()
    c.norm.weight.data.uniform_(0.5, 1.5)
    c.allocate_state(3, "cpu")
    from vllm_metax_b200.layers.basic import get_rope

    cs = get_rope(64, 64, 512, 10000.0, False).cos_sin_cache
    lengths = [300, 45]
    xs = [torch.randn(L, cfg.hidden_size) for L in lengths]
    got = [dict(), dict()]
    for parts in _steps(lengths, [(7, 3), (130, 1), (1, 1), (1, 40), (161, 0)]):
        md, pos = _metadata(parts, [[0, 1, 2], [3]], 128)
        x = torch.cat([xs[i][s:s + n] for i, s, n in parts])
        with set_forward_context(ForwardContext(attn_metadata=md, kv_caches=[])):
            entry, end, idx = c(x, pos, cs)
        o = 0
        for i, s, n in parts:
            for t in range(n):
                if end[o + t]:
                    got[i][int(idx[o + t])] = entry[o + t]
            o += n
    for i, L in enumerate(lengths):
        pooled = naive_compress(c.fused_wkv_wgate(xs[i]), c.ape, ratio, 128)
        assert sorted(got[i]) == list(range(L // ratio))
        if L // ratio == 0:
            continue
        want = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * c.norm.weight
        want = rope_tail(want, torch.arange(L // ratio) * ratio, cs, 64)
        torch.testing.assert_close(torch.stack([got[i][j] for j in range(L // ratio)]), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("layer,topk", [(0, 64), (0, 3), (1, 0), (2, 0)])
def test_v4_attention_layer_matches_per_token_oracle(layer, topk):
    """Layer 0: ratio 4 with the indexer (top-k >= entries = every entry, and a small top-k checked on the set the
    layer picked), layer 1: ratio 128 dense, layer 2: window only."""
    torch.manual_seed(1)
    cfg = _cfg(index_topk=topk or 4)
    attn = DeepseekV4Attention(cfg, 0, f"model.layers.{layer}.attn")
    for p in attn.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.15)
    for m in attn.modules():
        if isinstance(m, V4Compressor):
            m.ape.data.normal_()
    attn.attn_sink.data.copy_(torch.tensor([0.3, -0.5]))
    bs, lengths = 128, [270, 20]
    blocks = [[2, 0, 3], [1]]
    caches = [attn.allocate_kv_cache(4, bs, torch.float32, "cpu")]
    attn.allocate_state(3, "cpu")
    xs = [torch.randn(L, cfg.hidden_size) for L in lengths]
    outs = [[None] * L for L in lengths]
    picked = [[None] * L for L in lengths]
    for parts in _steps(lengths, [(100, 1), (30, 7), (1, 1), (139, 11)]):
        md, pos = _metadata(parts, blocks, bs)
        x = torch.cat([xs[i][s:s + n] for i, s, n in parts])
        with set_forward_context(ForwardContext(attn_metadata=md, kv_caches=caches)):
            y = attn(pos, x)
        o = 0
        for i, s, n in parts:
            for t in range(n):
                outs[i][s + t] = y[o + t]
                if attn.indexer is not None:
                    picked[i][s + t] = attn.last_selected[o + t]
            o += n
    cs, D = attn.rope.cos_sin_cache, 512
    for i, L in enumerate(lengths):
        x = xs[i]
        ar = torch.arange(L)
        qr_kv = attn.fused_wqa_wkv(x)
        qr, kv = attn.q_norm(qr_kv[:, : attn.q_lora].contiguous()), attn.kv_norm(qr_kv[:, attn.q_lora:].contiguous())
        q = attn.wq_b(qr).view(L, attn.heads, D)
        q = rope_tail(q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + attn.eps), ar, cs, 64)
        kv = rope_tail(kv, ar, cs, 64)
        comp = None
        if attn.ratio > 1:
            c = attn.compressor
            pooled = naive_compress(c.fused_wkv_wgate(x), c.ape, attn.ratio, D)
            if pooled.shape[0]:
                comp = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * c.norm.weight
                comp = rope_tail(comp, torch.arange(pooled.shape[0]) * attn.ratio, cs, 64)
        for p in range(L):
            sel = None
            if attn.indexer is not None:
                sel = picked[i][p]
                n_c = (p + 1) // attn.ratio
                assert int((sel >= 0).sum()) == min(n_c, attn.indexer.topk) and bool((sel < n_c).all())
                assert len(set(sel[sel >= 0].tolist())) == int((sel >= 0).sum())
            o = naive_v4_attention(q[p], kv, comp if comp is not None else torch.zeros(0, D), p, attn.window, attn.ratio,
                                   attn.scale, attn.attn_sink, sel)
            o = rope_tail(o[None], torch.tensor([p]), cs, 64, inverse=True)[0]
            G = attn.groups
            z = torch.einsum("gk,grk->gr", o.reshape(G, -1), attn.wo_a.weight.view(G, attn.o_lora, -1))
            want = attn.wo_b(z.reshape(1, -1))[0]
            torch.testing.assert_close(outs[i][p], want, rtol=2e-3, atol=2e-4, msg=lambda m: f"req {i} pos {p}: {m}")


def test_v4_model_with_compressed_attention_is_chunk_invariant_cpu():
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=16, block_size=128, max_model_len=384, seed=0)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 64, (n,), generator=g).tolist() for n in (150, 9, 261)]
    a = LLM(_cfg(), max_num_batched_tokens=512, **kw)
    assert a.engine.runner.model.v4_attention and a.engine.runner.state_slots is not None
    b = LLM(_cfg(), max_num_batched_tokens=37, **kw)
    b.engine.runner.model.load_state_dict(a.engine.runner.model.state_dict())
    ta = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    tb = [o.outputs[0].token_ids for o in b.generate(list(reversed(prompts)), sp)]
    assert ta == list(reversed(tb))
    assert all(len(t) == 6 for t in ta)


def _drive(attn, cfg, xs, lengths, blocks, bs, device, dtype):
    caches = [attn.allocate_kv_cache(4, bs, dtype, device)]
    attn.allocate_state(3, device)
    outs = [torch.zeros(L, cfg.hidden_size) for L in lengths]
    for parts in _steps(lengths, [(100, 1), (30, 7), (1, 1), (139, 11)]):
        md, pos = _metadata(parts, blocks, bs)
        for k in ("query_start_loc", "seq_lens", "block_table", "slot_mapping"):
            setattr(md, k, getattr(md, k).to(device))
        md.extra["state_indices"] = md.extra["state_indices"].to(device)
        x = torch.cat([xs[i][s:s + n] for i, s, n in parts]).to(device, dtype)
        with set_forward_context(ForwardContext(attn_metadata=md, kv_caches=caches)):
            y = attn(pos.to(device), x)
        o = 0
        for i, s, n in parts:
            outs[i][s:s + n] = y[o:o + n].float().cpu()
            o += n
    return outs


@pytest.mark.gpu
@pytest.mark.parametrize("layer", [0, 1, 2])
def test_v4_attention_layer_gpu_matches_cpu(layer, kernel_status_ok):
    """The same layer and steps on the device (bf16, CUDA latent-attention / cache / indexer kernels) and on the CPU
    reference ops (fp32 arithmetic on the same bf16 weights).  The ratio-4 layer keeps every entry (top-k >= entries)
    so that both sides attend the same set."""
    torch.manual_seed(2)
    cfg = _cfg(index_topk=80, index_n_heads=16, dtype=torch.bfloat16)
    with torch.device("cuda"):
        dev_attn = DeepseekV4Attention(cfg, 0, f"model.layers.{layer}.attn")
    cpu_cfg = _cfg(index_topk=80, index_n_heads=16, dtype=torch.float32)
    cpu_attn = DeepseekV4Attention(cpu_cfg, 0, f"model.layers.{layer}.attn")
    for p in dev_attn.parameters():
        if p.dim() >= 2:
            torch.nn.init.normal_(p, std=0.15)
    for m in dev_attn.modules():
        if isinstance(m, V4Compressor):
            m.ape.data.normal_()
    dev_attn.attn_sink.data.copy_(torch.tensor([0.3, -0.5], device="cuda"))
    cpu_attn.load_state_dict({k: v.float().cpu() for k, v in dev_attn.state_dict().items()})
    bs, lengths, blocks = 128, [270, 20], [[2, 0, 3], [1]]
    xs = [torch.randn(L, cfg.hidden_size).bfloat16().float() for L in lengths]
    got = _drive(dev_attn, cfg, xs, lengths, blocks, bs, "cuda", torch.bfloat16)
    want = _drive(cpu_attn, cpu_cfg, xs, lengths, blocks, bs, "cpu", torch.float32)
    for g, w in zip(got, want):
        cos = 1.0 - float(torch.nn.functional.cosine_similarity(g.flatten(), w.flatten(), dim=0))
        assert cos < 2e-3, cos
