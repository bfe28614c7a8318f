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
