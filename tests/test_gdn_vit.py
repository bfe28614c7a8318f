"""Gated delta rule (recurrent kernel vs the fp32 recurrence) and bidirectional encoder attention."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

gpu = pytest.mark.gpu


def _gdn_case(dtype, seed=0, Hq=2, Hv=4, lens=(5, 1, 33)):
    g_ = torch.Generator().manual_seed(seed)
    T = sum(lens)
    q = torch.randn(T, Hq, 128, generator=g_).to(dtype)
    k = torch.randn(T, Hq, 128, generator=g_).to(dtype)
    v = torch.randn(T, Hv, 128, generator=g_).to(dtype)
    g = -torch.rand(T, Hv, generator=g_) * 0.5
    beta = torch.rand(T, Hv, generator=g_)
    qsl = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    state = torch.randn(4, Hv, 128, 128, generator=g_) * 0.1
    idx = torch.tensor([2, 0, 3], dtype=torch.int32)
    has = torch.tensor([1, 0, 1], dtype=torch.int32)
    return q, k, v, g, beta, qsl, state, idx, has


def test_gdn_reference_properties():
    from vllm_metax_b200.ops.gdn import gated_delta_rule

    q, k, v, g, beta, qsl, state, idx, has = _gdn_case(torch.float32)
    s1 = state.clone()
    o_all = gated_delta_rule(q, k, v, g, beta, qsl, s1, idx, has)
    # the same tokens fed in two calls (chunked prefill) continue from the stored state
    s2 = state.clone()
    cut = torch.tensor([0, 3, 4, 20], dtype=torch.int32)                  # first 3 / 1 / 16 tokens of each sequence
    first = torch.cat([torch.arange(0, 3), torch.arange(5, 6), torch.arange(6, 22)])
    o_a = gated_delta_rule(q[first], k[first], v[first], g[first], beta[first], cut, s2, idx, has)
    rest = torch.cat([torch.arange(3, 5), torch.arange(22, 39)])
    cut2 = torch.tensor([0, 2, 2, 19], dtype=torch.int32)
    o_b = gated_delta_rule(q[rest], k[rest], v[rest], g[rest], beta[rest], cut2, s2, idx, torch.ones(3, dtype=torch.int32))
    torch.testing.assert_close(o_a, o_all[first], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(o_b, o_all[rest], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s2, s1, rtol=1e-4, atol=1e-4)
    assert torch.equal(s1[1], state[1])                                   # an unused slot is untouched


@pytest.mark.parametrize("lens,chunk", [((5, 1, 33), 64), ((200, 64, 129), 64), ((70, 3, 17), 16)])
def test_gdn_chunked_form_equals_the_recurrence(lens, chunk):
    """The matrix form over chunks (what prefill uses when switched on) against the token-by-token recurrence:
    sequences shorter than, equal to and not a multiple of the chunk, initial states, stored final states."""
    from vllm_metax_b200.ops.gdn import gated_delta_rule_chunked, gated_delta_rule_ref

    q, k, v, g, beta, qsl, state, idx, has = _gdn_case(torch.float32, seed=4, lens=lens)
    s_ref, s_chk = state.clone(), state.clone()
    want = gated_delta_rule_ref(q, k, v, g, beta, qsl, s_ref, idx, has)
    got = gated_delta_rule_chunked(q, k, v, g, beta, qsl, s_chk, idx, has, chunk=chunk)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(s_chk, s_ref, rtol=2e-4, atol=2e-4)
    assert torch.equal(s_chk[1], state[1])
    # strong decay and beta = 1 (the stiffest case for the triangular solve)
    g2, b2 = g * 8, torch.ones_like(beta)
    s_ref, s_chk = state.clone(), state.clone()
    want = gated_delta_rule_ref(q, k, v, g2, b2, qsl, s_ref, idx, has)
    got = gated_delta_rule_chunked(q, k, v, g2, b2, qsl, s_chk, idx, has, chunk=chunk)
    torch.testing.assert_close(got, want, rtol=5e-4, atol=5e-4)


def test_gdn_dispatch_takes_the_chunked_form_when_switched_on(monkeypatch):
    from vllm_metax_b200.ops import gdn

    q, k, v, g, beta, qsl, state, idx, has = _gdn_case(torch.float32, seed=2, lens=(300, 2, 40))
    calls = []
    real = gdn.gated_delta_rule_chunked
    monkeypatch.setattr(gdn, "gated_delta_rule_chunked", lambda *a, **kw: (calls.append(1), real(*a, **kw))[1])
    s0 = state.clone()
    want = gdn.gated_delta_rule(q, k, v, g, beta, qsl, s0, idx, has)
    assert not calls
    monkeypatch.setenv("B200_GDN_CHUNKED", "1")
    s1 = state.clone()
    got = gdn.gated_delta_rule(q, k, v, g, beta, qsl, s1, idx, has)
    assert calls == [1]
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(s1, s0, rtol=2e-4, atol=2e-4)
    short = torch.tensor([0, 5, 6, 39], dtype=torch.int32)                # no long chunk in the batch: recurrent
    gdn.gated_delta_rule(q[:39], k[:39], v[:39], g[:39], beta[:39], short, state.clone(), idx, has)
    assert calls == [1]


@gpu
def test_gdn_kernel_matches_reference():
    from vllm_metax_b200.ops.gdn import gated_delta_rule, gated_delta_rule_ref

    q, k, v, g, beta, qsl, state, idx, has = _gdn_case(torch.bfloat16, seed=1)
    s_ref = state.clone()
    want = gated_delta_rule_ref(q, k, v, g, beta, qsl, s_ref, idx, has)
    s_gpu = state.clone().cuda()
    got = gated_delta_rule(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), qsl.cuda(), s_gpu, idx.cuda(), has.cuda())
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(s_gpu.cpu(), s_ref, rtol=2e-3, atol=2e-3)
    # no state pool: every sequence starts from zero and nothing is stored
    o2 = gated_delta_rule(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), qsl.cuda())
    w2 = gated_delta_rule_ref(q, k, v, g, beta, qsl)
    torch.testing.assert_close(o2.float().cpu(), w2.float(), rtol=3e-2, atol=3e-2)


def _vit_ref(q, k, v, cu, scale):
    out = torch.zeros_like(q, dtype=torch.float32)
    for a, b in zip(cu[:-1].tolist(), cu[1:].tolist()):
        s = torch.einsum("qhd,khd->hqk", q[a:b].float(), k[a:b].float()) * scale
        out[a:b] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v[a:b].float())
    return out


def test_encoder_attention_cpu():
    from vllm_metax_b200.layers.mm_encoder_attention import MMEncoderAttention

    g = torch.Generator().manual_seed(0)
    H, D = 4, 64
    cu = torch.tensor([0, 9, 9 + 16, 9 + 16 + 5], dtype=torch.int32)
    q, k, v = (torch.randn(30, H * D, generator=g) for _ in range(3))
    attn = MMEncoderAttention(H, D)
    out = attn(q, k, v, cu, 16)
    want = _vit_ref(q.view(30, H, D), k.view(30, H, D), v.view(30, H, D), cu, D ** -0.5)
    torch.testing.assert_close(out.float(), want, rtol=1e-4, atol=1e-4)
    # batched [B, S, H, D] form without cu_seqlens: every image is one sequence
    qb = torch.randn(2, 7, H, D, generator=g)
    ob = attn(qb, qb, qb)
    wb = _vit_ref(qb.reshape(14, H, D), qb.reshape(14, H, D), qb.reshape(14, H, D), torch.tensor([0, 7, 14]), D ** -0.5)
    torch.testing.assert_close(ob.reshape(14, H, D).float(), wb, rtol=1e-4, atol=1e-4)


@gpu
@pytest.mark.parametrize("D", [64, 128])
def test_encoder_attention_gpu(D):
    from vllm_metax_b200.layers.mm_encoder_attention import MMEncoderAttention

    g = torch.Generator().manual_seed(1)
    H = 8
    lens = [200, 64, 1, 333]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    T = sum(lens)
    q, k, v = (torch.randn(T, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    out = MMEncoderAttention(H, D)(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), max(lens))
    torch.testing.assert_close(out.float().cpu(), _vit_ref(q, k, v, cu, D ** -0.5), rtol=3e-2, atol=3e-2)


# ------------------------------------------------------------------------------------------ short causal convolution
def _conv_case(dtype, seed=0, C=384, K=4, lens=(5, 1, 70, 2)):
    g_ = torch.Generator().manual_seed(seed)
    T = sum(lens)
    x = torch.randn(T, C + 64, generator=g_).to(dtype)[:, :C]            # row pitch larger than C
    w = (torch.randn(C, K, generator=g_) * 0.5).to(dtype)
    bias = (torch.randn(C, generator=g_) * 0.1).to(dtype)
    qsl = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    state = torch.randn(6, K - 1, C, generator=g_).to(dtype)
    idx = torch.tensor([4, 1, 0, 5], dtype=torch.int32)
    has = torch.tensor([1, 1, 0, 1], dtype=torch.int32)
    return x, w, bias, qsl, state, idx, has


def test_causal_conv1d_reference_is_a_streaming_convolution():
    """Feeding a sequence in pieces through the carry gives the same outputs as feeding it at once."""
    from vllm_metax_b200.ops.gdn import causal_conv1d

    x, w, bias, *_ = _conv_case(torch.float32, lens=(40,))
    one = torch.tensor([0], dtype=torch.int32)
    whole = causal_conv1d(x, w, bias, torch.zeros(1, 3, x.shape[1]), torch.tensor([0, 40], dtype=torch.int32), one,
                          torch.tensor([0], dtype=torch.int32))
    st = torch.zeros(1, 3, x.shape[1])
    parts, pos = [], 0
    for n in (1, 2, 17, 1, 19):
        parts.append(causal_conv1d(x[pos:pos + n], w, bias, st, torch.tensor([0, n], dtype=torch.int32), one,
                                   torch.tensor([1 if pos else 0], dtype=torch.int32)))
        pos += n
    torch.testing.assert_close(torch.cat(parts), whole, atol=1e-5, rtol=1e-5)
    # and against torch's own depthwise convolution
    ref = torch.nn.functional.conv1d(x.t()[None], w[:, None], bias, padding=3, groups=x.shape[1])[0, :, :40].t()
    torch.testing.assert_close(whole, torch.nn.functional.silu(ref), atol=1e-5, rtol=1e-5)


@gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("K", [2, 4])
def test_causal_conv1d_kernel_matches_reference(dtype, K):
    from vllm_metax_b200.ops.gdn import causal_conv1d, causal_conv1d_ref

    x, w, bias, qsl, state, idx, has = _conv_case(dtype, K=K)
    st_ref = state.clone()
    want = causal_conv1d_ref(x, w, bias, st_ref, qsl, idx, has)
    st = state.cuda()
    got = causal_conv1d(x.cuda(), w.cuda(), bias.cuda(), st, qsl.cuda(), idx.cuda(), has.cuda())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol, rtol=tol)
    torch.testing.assert_close(st.float().cpu(), st_ref.float(), atol=0, rtol=0)          # carries are copies of inputs
    # no carry: every sequence starts from zeros and nothing is written back
    got2 = causal_conv1d(x.cuda(), w.cuda(), None, None, qsl.cuda(), None, None, silu=False)
    want2 = causal_conv1d_ref(x, w, None, None, qsl, None, None, silu=False)
    torch.testing.assert_close(got2.float().cpu(), want2.float(), atol=tol, rtol=tol)


@gpu
def test_qwen3_next_engine_on_gpu_graphs_match_eager():
    """Hybrid model end to end on the GPU kernels (delta-rule head size 128, attention head size 128): decode steps
    replayed from CUDA graphs must give the tokens of the eager run, with requests spread over several state slots."""
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200.config import ModelConfig

    hf = dict(architectures=["Qwen3NextForCausalLM"], vocab_size=1024, hidden_size=256, num_hidden_layers=4,
              num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512,
              intermediate_size=512, moe_intermediate_size=128, shared_expert_intermediate_size=128, num_experts=8,
              num_experts_per_tok=2, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=128,
              linear_value_head_dim=128, linear_conv_kernel_dim=4, norm_topk_prob=True, torch_dtype="bfloat16")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (37, 5, 130, 64, 9)]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    outs = []
    for eager in (True, False):
        llm = LLM(ModelConfig.from_hf_dict(hf, seed=3), max_model_len=256, max_num_seqs=4, max_num_batched_tokens=128,
                  num_gpu_blocks=64, enforce_eager=eager, load_format="dummy")
        outs.append([list(o.outputs[0].token_ids) for o in llm.generate(prompts, sp)])
        assert not llm.engine.runner.state_slots
        del llm
        torch.cuda.empty_cache()
    assert outs[0] == outs[1]
    assert all(len(t) == 12 for t in outs[0])
