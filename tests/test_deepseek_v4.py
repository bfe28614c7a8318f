"""DeepSeek-V4 pieces: mHC kernels vs the fp32 statement, name rewriting, and the model end to end on CPU."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200.ops import mhc

gpu = pytest.mark.gpu


def _cfg(**kw):
    base = dict(architecture="DeepseekV4ForCausalLM", vocab_size=64, hidden_size=128, intermediate_size=256,
                num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, q_lora_rank=64, kv_lora_rank=512,
                qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_experts=4, num_experts_per_tok=2,
                moe_intermediate_size=64, n_shared_experts=1, first_k_dense_replace=0, scoring_func="sqrtsoftplus",
                routed_scaling_factor=1.5, hc_mult=4, hc_sinkhorn_iters=5, num_hash_layers=1,
                max_position_embeddings=256, dtype=torch.float32)
    base.update(kw)
    return ModelConfig(**base)


def test_sinkhorn_is_doubly_stochastic():
    x = mhc.sinkhorn(torch.randn(7, 4, 4), 20, 1e-6)
    assert torch.allclose(x.sum(-2), torch.ones(7, 4), atol=1e-3) and torch.allclose(x.sum(-1), torch.ones(7, 4), atol=2e-2)


def test_fused_equals_post_then_pre_cpu():
    torch.manual_seed(0)
    T, M, H = 5, 4, 32
    res = torch.randn(T, M, H)
    fn, base, scale = torch.randn(24, M * H) * 0.05, torch.randn(24) * 0.1, torch.rand(3) + 0.5
    post, comb, x = mhc.mhc_pre(res, fn, scale, base, 1e-6, 1e-6, 1e-6, 2.0, 5)
    y = torch.randn(T, H)
    new_res, p2, c2, x2 = mhc.mhc_fused_post_pre(y, res, post, comb, fn, scale, base, 1e-6, 1e-6, 1e-6, 2.0, 5)
    want_res = mhc.mhc_post(y, res, post, comb)
    torch.testing.assert_close(new_res, want_res)
    p3, c3, x3 = mhc.mhc_pre(want_res, fn, scale, base, 1e-6, 1e-6, 1e-6, 2.0, 5)
    torch.testing.assert_close(x2, x3)
    torch.testing.assert_close(c2, c3)


def test_v4_weight_name_rewriting():
    from vllm_metax_b200.models.deepseek_v4 import rename_v4

    assert rename_v4("layers.3.attn.wq_a.weight") == "model.layers.3.attn.q_a_proj.weight"
    assert rename_v4("layers.0.ffn.experts.7.w1.weight") == "model.layers.0.ffn.experts.7.gate_proj.weight"
    assert rename_v4("layers.2.hc_attn_fn") == "model.layers.2.hc_attn.fn"
    assert rename_v4("head.weight") == "lm_head.weight"
    assert rename_v4("embed.weight") == "model.embed_tokens.weight"


def test_v4_model_generates_and_is_deterministic_cpu():
    kw = dict(device="cpu", load_format="dummy", num_gpu_blocks=16, block_size=64, max_model_len=128, seed=0)
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    a = LLM(_cfg(), **kw).generate([[1, 2, 3, 4], [5, 6]], sp)
    b = LLM(_cfg(), **kw).generate([[5, 6], [1, 2, 3, 4]], sp)
    assert a[0].outputs[0].token_ids == b[1].outputs[0].token_ids       # batch-order invariant
    assert len(a[1].outputs[0].token_ids) == 6


@gpu
@pytest.mark.parametrize("T,M,H", [(1, 4, 1024), (9, 4, 7168), (130, 2, 512)])
def test_mhc_kernels_gpu(T, M, H, kernel_status_ok):
    torch.manual_seed(1)
    nmix = (2 + M) * M
    res = torch.randn(T, M, H).bfloat16()
    fn, base, scale = torch.randn(nmix, M * H) * 0.02, torch.randn(nmix) * 0.1, torch.rand(3) + 0.5
    args = (1e-6, 1e-6, 1e-6, 2.0, 6)
    post, comb, x = mhc.mhc_pre(res, fn, scale, base, *args)
    gp, gc, gx = mhc.mhc_pre(res.cuda(), fn.cuda(), scale.cuda(), base.cuda(), *args)
    torch.testing.assert_close(gp.cpu(), post, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(gc.cpu(), comb, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(gx.float().cpu(), x.float(), rtol=2e-2, atol=2e-2)
    y = torch.randn(T, H).bfloat16()
    want = mhc.mhc_fused_post_pre(y, res, post, comb, fn, scale, base, *args)
    got = mhc.mhc_fused_post_pre(y.cuda(), res.cuda(), gp, gc, fn.cuda(), scale.cuda(), base.cuda(), *args)
    torch.testing.assert_close(got[0].float().cpu(), want[0].float(), rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(got[2].cpu(), want[2], rtol=5e-3, atol=5e-3)
    torch.testing.assert_close(got[3].float().cpu(), want[3].float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(mhc.mhc_post(y.cuda(), res.cuda(), gp, gc).float().cpu(), mhc.mhc_post(y, res, post, comb).float(),
                               rtol=2e-2, atol=3e-2)
    hfn, hbase, hscale = torch.randn(M, M * H) * 0.02, torch.randn(M) * 0.1, torch.rand(1) + 0.5
    torch.testing.assert_close(mhc.mhc_head(res.cuda(), hfn.cuda(), hscale.cuda(), hbase.cuda(), 1e-6, 1e-6).float().cpu(),
                               mhc.mhc_head(res, hfn, hscale, hbase, 1e-6, 1e-6).float(), rtol=2e-2, atol=2e-2)


@gpu
def test_v4_model_gpu_matches_cpu_tokens(kernel_status_ok):
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    cpu = LLM(_cfg(num_experts=8), device="cpu", load_format="dummy", num_gpu_blocks=16, block_size=64, max_model_len=128, seed=0)
    gpu_llm = LLM(_cfg(num_experts=8, dtype=torch.bfloat16), device="cuda", load_format="dummy", num_gpu_blocks=16, block_size=64,
                  max_model_len=128, seed=0)
    gpu_llm.engine.runner.model.load_state_dict({k: v for k, v in cpu.engine.runner.model.state_dict().items()}, strict=False)
    out = gpu_llm.generate([[1, 2, 3, 4]], sp)
    assert len(out[0].outputs[0].token_ids) == 5


# ------------------------------------------------------------------------------- latent-cache records
def _record_case(device, T=37, Hq=5, hq_pad=8, block_size=16, n_insert=33):
    from vllm_metax_b200.ops import v4_cache as vc

    g = torch.Generator().manual_seed(3)
    q = (torch.randn(T, Hq, 512, generator=g) * 2).to(torch.bfloat16).to(device)
    kv = (torch.randn(T, 512, generator=g) * torch.logspace(-3, 2, 512)).to(torch.bfloat16).to(device)
    pos = torch.randint(0, 300, (T,), generator=g).to(device)
    ang = torch.arange(300)[:, None].float() * (1.0 / 10000 ** (torch.arange(32).float() / 32))[None]
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).to(device)
    slots = torch.randperm(4 * block_size, generator=g)[:n_insert]
    slots[5] = -1
    cache = vc.alloc_cache(4, block_size, device)
    return vc, q, kv, pos, cos_sin, slots.to(device), cache, hq_pad, block_size


def test_v4_records_reference_round_trip():
    vc, q, kv, pos, cos_sin, slots, cache, hq_pad, bs = _record_case("cpu")
    q_out = vc.qnorm_rope_kv_insert(q, kv, cache, slots, pos, cos_sin, 1e-6, bs, hq_pad)
    assert q_out.shape == (37, hq_pad, 512) and q_out[:, 5:].abs().max() == 0
    # normalised heads have unit RMS (RoPE is a rotation)
    torch.testing.assert_close(q_out[:, :5].float().pow(2).mean(-1), torch.ones(37, 5), rtol=2e-2, atol=2e-2)
    back = vc.gather_dequant(cache, slots, bs).float()
    rows = cos_sin[pos[: slots.numel()]]
    want = torch.cat([kv[: slots.numel(), :448].float(), vc._rope_interleaved(kv[: slots.numel(), 448:].float(), rows)], -1)
    live = slots >= 0
    assert back[~live].abs().max() == 0
    # e4m3 with a power-of-two scale per 64 values: 3 mantissa bits -> relative error up to 2^-4 of the block maximum
    err = (back[live] - want[live]).abs().view(-1, 8, 64).amax(-1)
    ref = want[live].abs().view(-1, 8, 64).amax(-1).clamp_min(1e-4)
    assert (err / ref).max() < 0.07
    torch.testing.assert_close(back[live][:, 448:], want[live][:, 448:].to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
def test_v4_records_kernel_matches_reference():
    vc, q, kv, pos, cos_sin, slots, cache, hq_pad, bs = _record_case("cuda")
    # q as a view with padded pitches, as it comes out of a fused projection
    q_wide = torch.zeros(q.shape[0], q.shape[1], 520, dtype=q.dtype, device="cuda")
    q_wide[..., :512] = q
    q_out = vc.qnorm_rope_kv_insert(q_wide[..., :512], kv, cache, slots, pos, cos_sin, 1e-6, bs, hq_pad)
    cache_ref = vc.alloc_cache(4, bs, "cpu")
    q_ref = vc.qnorm_rope_kv_insert_ref(q.cpu(), kv.cpu(), cache_ref, slots.cpu(), pos.cpu(), cos_sin.cpu(), 1e-6, bs, hq_pad)
    torch.testing.assert_close(q_out.float().cpu(), q_ref.float(), rtol=2e-2, atol=2e-2)
    got = vc.gather_dequant(cache, slots, bs).float().cpu()
    want = vc.gather_dequant_ref(cache_ref, slots.cpu(), bs).float()
    # identical scales except where an amax sits on a power-of-two boundary; compare dequantised values
    torch.testing.assert_close(got, want, rtol=0.13, atol=1e-3)
    same = (cache.cpu() == cache_ref).float().mean()
    assert same > 0.98, same
    # the kernel's own reader agrees with the PyTorch reader on the kernel's bytes
    torch.testing.assert_close(got, vc.gather_dequant_ref(cache.cpu(), slots.cpu(), bs).float(), rtol=0, atol=0)


def _cs64(n=300):
    ang = torch.arange(n)[:, None].float() * (1.0 / 10000 ** (torch.arange(32).float() / 32))[None]
    return torch.cat([ang.cos(), ang.sin()], -1)


def test_v4_inv_rope_undoes_the_insert_rotation():
    from vllm_metax_b200.ops import v4_cache as vc

    g = torch.Generator().manual_seed(5)
    T, H = 9, 4
    x = torch.randn(T, H, 512, generator=g)
    pos = torch.randint(0, 300, (T,), generator=g)
    cs = _cs64()
    rot = torch.cat([x[..., :448], vc._rope_interleaved(x[..., 448:], cs[pos][:, None, :])], -1)
    back = vc.inv_rope(rot, pos, cs, n_groups=2)
    assert back.shape == (T, 2, 2 * 512)
    torch.testing.assert_close(back.reshape(T, H, 512), x, rtol=1e-5, atol=1e-5)


def test_v4_indexer_q_reference_contract():
    from vllm_metax_b200.ops import v4_cache as vc

    g = torch.Generator().manual_seed(6)
    T, H = 7, 3
    q = torch.randn(T, H, 128, generator=g)
    w = torch.randn(T, H, generator=g)
    pos = torch.randint(0, 300, (T,), generator=g)
    q8, w_out = vc.indexer_q_rope_int8_quant(pos, q, _cs64(), w, 0.5, 0.25)
    assert q8.dtype == torch.int8 and q8.abs().max() == 127
    # q8 * folded weight reproduces (rotated q) * w * softmax_scale * head_scale
    want = torch.cat([q[..., :64], vc._rope_interleaved(q[..., 64:], _cs64()[pos][:, None, :])], -1)
    got = q8.float() * (w_out / (w * 0.125))[..., None]
    torch.testing.assert_close(got, want, rtol=0, atol=float(want.abs().max()) / 127 + 1e-2)


@pytest.mark.gpu
def test_v4_inv_rope_and_indexer_q_kernels():
    from vllm_metax_b200.ops import v4_cache as vc

    g = torch.Generator().manual_seed(7)
    T, H = 45, 8
    cs = _cs64()
    pos = torch.randint(0, 300, (T,), generator=g)
    o = torch.randn(T, H, 512, generator=g).to(torch.bfloat16)
    wide = torch.zeros(T, H, 528, dtype=torch.bfloat16, device="cuda")
    wide[..., :512] = o.cuda()
    got = vc.inv_rope(wide[..., :512], pos.cuda(), cs.cuda(), n_groups=4)
    want = vc.inv_rope(o, pos, cs, n_groups=4)
    assert got.shape == want.shape
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=2e-2, atol=2e-2)
    q = torch.randn(T, H, 128, generator=g).to(torch.bfloat16)
    w = torch.randn(T, H, generator=g).to(torch.bfloat16)
    q8, w_out = vc.indexer_q_rope_int8_quant(pos.cuda(), q.cuda(), cs.cuda(), w.cuda(), 0.5, 0.25)
    q8_ref, w_ref = vc.indexer_q_rope_int8_quant(pos, q, cs, w, 0.5, 0.25)
    torch.testing.assert_close(w_out.cpu(), w_ref, rtol=1e-2, atol=1e-5)
    assert (q8.cpu().int() - q8_ref.int()).abs().max() <= 1
    assert (q8.cpu() == q8_ref).float().mean() > 0.97
