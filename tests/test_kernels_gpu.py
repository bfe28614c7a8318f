"""CUDA kernels vs the fp32 PyTorch reference of the same op (run on a B200)."""
import math

import pytest
import torch

from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cos_diff(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


@pytest.fixture(autouse=True)
def _status(kernel_status_ok):
    yield


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 1536, 4096), (4096, 6144, 4096),
                                   (333, 264, 520), (129, 4096, 14336)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_tcgen05(M, N, K, dtype):
    a = torch.randn(M, K, device=DEV, dtype=dtype)
    w = torch.randn(N, K, device=DEV, dtype=dtype) * 0.05
    want = (a.float() @ w.float().t())
    got = ops.gemm(a, w)
    torch.cuda.synchronize()
    assert got.shape == (M, N)
    err = (got.float() - want).abs().max() / want.abs().max()
    assert err < 1.5e-2, err
    assert cos_diff(got, want) < 1e-5


@pytest.mark.parametrize("force_bn", [256, 128, 64, 32, -16, -32, -64])
def test_gemm_every_tile_config(force_bn):
    M = 48 if force_bn < 0 else 300
    N, K = 1280, 1024
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    want = a.float() @ w.float().t() + bias.float() + res.float()
    got = ops.gemm(a, w, bias, res, force_bn=force_bn)
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2


@pytest.mark.parametrize("M", [1, 7, 16, 33, 64])
def test_gemm_small_m_swap(M):
    a = torch.randn(M, 4096, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(6144, 4096, device=DEV, dtype=torch.bfloat16) * 0.05
    want = a.float() @ w.float().t()
    got = ops.gemm(a, w)
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2


def test_gemm_strided_input_view():
    big = torch.randn(200, 3 * 512, device=DEV, dtype=torch.bfloat16)
    a = big[:, 512:1024]
    w = torch.randn(384, 512, device=DEV, dtype=torch.bfloat16) * 0.05
    want = a.float() @ w.float().t()
    assert (ops.gemm(a, w).float() - want).abs().max() / want.abs().max() < 1.5e-2


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("T,H", [(1, 256), (7, 4096), (300, 8192), (5, 7168), (3, 520)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rms_norm(T, H, dtype):
    x = torch.randn(T, H, device=DEV, dtype=dtype)
    w = torch.randn(H, device=DEV, dtype=dtype)
    torch.testing.assert_close(ops.rms_norm(x, w, 1e-5), ref.rms_norm(x, w, 1e-5), rtol=2e-2, atol=2e-2)
    r = torch.randn(T, H, device=DEV, dtype=dtype)
    wy, wr = ref.fused_add_rms_norm(x, r, w, 1e-5)
    x2, r2 = x.clone(), r.clone()
    ops.fused_add_rms_norm(x2, r2, w, 1e-5)
    torch.testing.assert_close(r2, wr, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(x2, wy, rtol=2e-2, atol=2e-2)


def test_head_rms_norm():
    T, H, D = 9, 6, 128
    x = torch.randn(T, H * D + 256, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(D, device=DEV, dtype=torch.bfloat16)
    want = ref.rms_norm(x[:, : H * D].reshape(T, H, D), w, 1e-6).reshape(T, -1)
    tail = x[:, H * D:].clone()
    ops.head_rms_norm(x, w, 1e-6, H, D)
    torch.testing.assert_close(x[:, : H * D], want, rtol=2e-2, atol=2e-2)
    assert torch.equal(x[:, H * D:], tail)


@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm_quant_variants(with_res):
    T, H = 11, 2048
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(H, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(T, H, device=DEV, dtype=torch.bfloat16) if with_res else None
    # per-token fp8
    q, s = ops.rms_norm_dynamic_per_token_quant(x, w, 1e-5, residual=None if res is None else res.clone())
    wq, ws, _ = ref.rms_norm_dynamic_per_token_quant(x, w, 1e-5, residual=res)
    torch.testing.assert_close(s, ws, rtol=2e-2, atol=1e-6)
    assert cos_diff(q.float() * s, wq.float() * ws) < 1e-3
    # per-token int8
    q, s = ops.rms_norm_dynamic_per_token_quant(x, w, 1e-5, torch.int8, residual=None if res is None else res.clone())
    wq, ws, _ = ref.rms_norm_dynamic_per_token_quant(x, w, 1e-5, torch.int8, residual=res)
    assert cos_diff(q.float() * s, wq.float() * ws) < 1e-3
    # per-128 block fp8
    q, s = ops.rms_norm_per_block_quant(x, w, 1e-5, 128, residual=None if res is None else res.clone())
    wq, ws, _ = ref.rms_norm_per_block_quant(x, w, 1e-5, 128, residual=res)
    torch.testing.assert_close(s, ws, rtol=2e-2, atol=1e-6)
    deq = (q.float().reshape(T, -1, 128) * s[..., None]).reshape(T, H)
    wdeq = (wq.float().reshape(T, -1, 128) * ws[..., None]).reshape(T, H)
    assert cos_diff(deq, wdeq) < 1e-3
    # static fp8
    sc = torch.tensor([0.02], device=DEV)
    q = ops.rms_norm_static_fp8_quant(x, w, sc, 1e-5)
    assert cos_diff(q.float(), ref.rms_norm_static_fp8_quant(x, w, sc, 1e-5).float()) < 1e-3


# ------------------------------------------------------------------ activations
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh", "relu2", "mul_silu", "swigluoai", "swiglustep"])
def test_act_and_mul(act):
    x = torch.randn(13, 2 * 1536, device=DEV, dtype=torch.bfloat16)
    got = ops.act_and_mul(x, act)
    want = ops.act_and_mul(x.cpu(), act).to(DEV)
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)


def test_silu_mul_block_quant():
    x = torch.randn(10, 2 * 1024, device=DEV, dtype=torch.bfloat16)
    q, s = ops.silu_and_mul_per_block_quant(x, 128)
    wq, ws = ref.silu_and_mul_per_block_quant(x, 128)
    torch.testing.assert_close(s, ws, rtol=2e-2, atol=1e-7)
    a = (q.float().reshape(10, -1, 128) * s[..., None])
    b = (wq.float().reshape(10, -1, 128) * ws[..., None])
    assert cos_diff(a, b) < 1e-3


# ------------------------------------------------------------------ rope + cache
@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("D,rot", [(128, 128), (64, 64), (128, 64), (256, 128)])
def test_rotary_embedding(neox, D, rot):
    T, Hq, Hk = 17, 8, 2
    q = torch.randn(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, Hk * D, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=DEV)
    cache = ref.build_rope_cache(rot, 512, 10000.0).to(DEV)
    wq, wk = ref.rotary_embedding(pos, q, k, D, cache, neox)
    ops.rotary_embedding(pos, q, k, D, cache, neox)
    torch.testing.assert_close(q, wq, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(k, wk, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kind", ["bf16", "fp8_static", "int8_per_token_head", "fp8_per_token_head"])
def test_rope_and_cache_write(kind):
    T, Hq, Hk, D, bs, nb = 40, 8, 2, 128, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D:(Hq + Hk) * D], qkv[:, (Hq + Hk) * D:]
    pos = torch.arange(T, device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[3] = -1
    cos_sin = ref.build_rope_cache(D, 64, 10000.0).to(DEV)
    dt = {"bf16": torch.bfloat16, "fp8_static": torch.float8_e4m3fn, "int8_per_token_head": torch.int8,
          "fp8_per_token_head": torch.float8_e4m3fn}[kind]
    cache = torch.zeros(nb, 2, bs, Hk, D, device=DEV, dtype=dt)
    scales = torch.ones(nb, 2, bs, Hk, device=DEV) if kind.endswith("head") else None
    wcache, wscales = cache.clone(), None if scales is None else scales.clone()
    wq, wk = ref.rotary_embedding(pos, q.contiguous(), k.contiguous(), D, cos_sin, True)
    ref.reshape_and_cache(wk.reshape(T, Hk, D), v.reshape(T, Hk, D), wcache, slots, wscales, 0.05, 0.07)
    ops.rope_and_cache(pos, q, k, v, D, cos_sin, True, cache, slots, scales, 0.05, 0.07)
    torch.testing.assert_close(q, wq, rtol=2e-2, atol=2e-2)
    if scales is not None:
        torch.testing.assert_close(scales, wscales, rtol=1e-2, atol=1e-6)
        assert cos_diff(cache.float() * scales[..., None], wcache.float() * wscales[..., None]) < 2e-3
    else:
        assert cos_diff(cache.float(), wcache.float()) < 2e-3


def test_concat_and_cache_mla_both_formats():
    T, bs, nb = 19, 64, 4
    kv_c = torch.randn(T, 512, device=DEV, dtype=torch.bfloat16)
    k_pe = torch.randn(T, 64, device=DEV, dtype=torch.bfloat16)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    c = torch.zeros(nb, bs, 576, device=DEV, dtype=torch.bfloat16)
    wc = c.clone()
    ops.concat_and_cache_mla(kv_c, k_pe, c, slots)
    ref.concat_and_cache_mla(kv_c, k_pe, wc, slots)
    assert torch.equal(c, wc)
    c8 = torch.zeros(nb, bs, 656, device=DEV, dtype=torch.uint8)
    w8 = c8.clone()
    ops.concat_and_cache_mla(kv_c, k_pe, c8, slots)
    ref.concat_and_cache_mla(kv_c, k_pe, w8, slots)
    a, b = ref.unpack_ds_mla(c8.reshape(-1, 656)), ref.unpack_ds_mla(w8.reshape(-1, 656))
    assert cos_diff(a, b) < 1e-4
    assert torch.equal(c8[..., 528:], w8[..., 528:])


def test_indexer_k_quant_and_cache():
    T, bs, nb = 33, 64, 3
    k = torch.randn(T, 128, device=DEV, dtype=torch.bfloat16)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    c = torch.zeros(nb, bs * 132, device=DEV, dtype=torch.uint8)
    w = c.clone()
    ops.indexer_k_quant_and_cache(k, c, slots, bs)
    ref.indexer_k_quant_and_cache(k, w, slots)
    bt = torch.arange(nb, device=DEV, dtype=torch.int32)
    kq, sc = ref.gather_indexer_k(c, bt, nb * bs)
    wq, wsc = ref.gather_indexer_k(w, bt, nb * bs)
    torch.testing.assert_close(sc, wsc, rtol=1e-3, atol=1e-8)
    assert cos_diff(kq * sc[:, None], wq * wsc[:, None]) < 1e-4


def test_copy_blocks():
    c = torch.randn(10, 2, 16, 2, 64, device=DEV, dtype=torch.bfloat16)
    w = c.clone()
    pairs = torch.tensor([[0, 5], [1, 7], [2, 9]], device=DEV)
    ops.copy_blocks([c], pairs)
    ref.copy_blocks([w], pairs)
    assert torch.equal(c, w)


# ------------------------------------------------------------------ attention
def make_paged(B, lens, Hkv, D, bs, dtype, kind="same", extra_blocks=3):
    """Random paged cache + block tables for sequences of the given kv lengths."""
    nblk = [(l + bs - 1) // bs for l in lens]
    total = sum(nblk) + extra_blocks
    perm = torch.randperm(total)
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o:o + nblk[b]].to(torch.int32)
        o += nblk[b]
    kv = torch.randn(total, 2, bs, Hkv, D)
    scales = None
    if kind == "same":
        cache = kv.to(dtype)
    elif kind == "int8":
        sc = kv.abs().amax(-1) / 127.0
        cache = torch.round(kv / sc[..., None]).clamp(-128, 127).to(torch.int8)
        scales = sc.float()
    elif kind == "fp8":
        sc = kv.abs().amax(-1) / 448.0
        cache = (kv / sc[..., None]).to(torch.float8_e4m3fn)
        scales = sc.float()
    return cache.to(DEV), (None if scales is None else scales.to(DEV)), bt.to(DEV)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 8, 64), (16, 2, 128), (4, 1, 256)])
@pytest.mark.parametrize("bs", [16, 64])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode(Hq, Hkv, D, bs, splits):
    lens = [1, 17, 300, 1025, 64]
    B = len(lens)
    cache, _, bt = make_paged(B, lens, Hkv, D, bs, torch.bfloat16)
    q = torch.randn(B, Hq, D, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    got = ops.paged_attention_decode(q, cache, bt, sl, scale, num_splits=splits)
    qsl = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    want = ref.paged_attention(q, cache, bt, sl, qsl, scale)
    assert cos_diff(got, want) < 2e-4
    torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("kind", ["int8", "fp8"])
def test_paged_decode_quantised_kv(kind):
    Hq, Hkv, D, bs = 32, 8, 128, 16
    lens = [5, 130, 777]
    cache, scales, bt = make_paged(3, lens, Hkv, D, bs, torch.bfloat16, kind)
    q = torch.randn(3, Hq, D, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = ops.paged_attention_decode(q, cache, bt, sl, D ** -0.5, kv_scales=scales, num_splits=2)
    want = ref.paged_attention(q, cache, bt, sl, torch.arange(4, dtype=torch.int32, device=DEV), D ** -0.5,
                               kv_scales=scales)
    assert cos_diff(got, want) < 5e-4


def test_paged_decode_window_softcap_sinks_multitoken():
    Hq, Hkv, D, bs = 8, 2, 128, 16
    lens = [40, 200]
    qlens = [3, 2]
    cache, _, bt = make_paged(2, lens, Hkv, D, bs, torch.bfloat16)
    T = sum(qlens)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    qsl = torch.tensor([0, 3, 5], dtype=torch.int32, device=DEV)
    sinks = torch.randn(Hq, device=DEV)
    lse = torch.empty(Hq, T, device=DEV)
    got = ops.paged_attention_decode(q, cache, bt, sl, D ** -0.5, query_start_loc=qsl, max_q_len=3, window=64,
                                     softcap=30.0, sinks=sinks, lse_out=lse, num_splits=1)
    want = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, window=64, softcap=30.0, sinks=sinks)
    assert cos_diff(got, want) < 3e-4


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 4, 64), (28, 4, 128)])
@pytest.mark.parametrize("bs", [16, 64, 128])
def test_prefill_tcgen05_paged(Hq, Hkv, D, bs):
    # (q_len, kv_len): pure prefill, chunked prefill with context, short and ragged cases
    cases = [(200, 200), (64, 300), (1, 1), (129, 129), (257, 1000)]
    lens = [c[1] for c in cases]
    B = len(cases)
    cache, _, bt = make_paged(B, lens, Hkv, D, bs, torch.bfloat16)
    T = sum(c[0] for c in cases)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    qsl = torch.tensor([0] + list(torch.tensor([c[0] for c in cases]).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    lse = torch.empty(Hq, T, device=DEV)
    got = ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, max_q_len=257, lse_out=lse)
    want, wlse = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, return_lse=True)
    assert cos_diff(got, want) < 3e-4
    torch.testing.assert_close(got.float(), want.float(), rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(lse, wlse, rtol=2e-2, atol=2e-2)


def test_prefill_window_softcap_sinks():
    Hq, Hkv, D, bs = 8, 2, 128, 64
    cases = [(300, 300), (100, 400)]
    lens = [c[1] for c in cases]
    cache, _, bt = make_paged(2, lens, Hkv, D, bs, torch.bfloat16)
    q = torch.randn(400, Hq, D, device=DEV, dtype=torch.bfloat16)
    qsl = torch.tensor([0, 300, 400], dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    sinks = torch.randn(Hq, device=DEV)
    got = ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, max_q_len=300, window=128, softcap=50.0,
                                      sinks=sinks)
    want = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, window=128, softcap=50.0, sinks=sinks)
    assert cos_diff(got, want) < 3e-4


def test_prefill_quantised_cache_falls_to_split_kernel():
    Hq, Hkv, D, bs = 16, 4, 128, 16
    cases = [(50, 50), (20, 90)]
    lens = [c[1] for c in cases]
    cache, scales, bt = make_paged(2, lens, Hkv, D, bs, torch.bfloat16, "int8")
    q = torch.randn(70, Hq, D, device=DEV, dtype=torch.bfloat16)
    qsl = torch.tensor([0, 50, 70], dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, kv_scales=scales, max_q_len=50)
    want = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, kv_scales=scales)
    assert cos_diff(got, want) < 5e-4


@pytest.mark.parametrize("dqk,dv", [(128, 128), (192, 128)])
def test_varlen_attention_contiguous(dqk, dv):
    H = 16
    lq, lk = [100, 37, 256], [100, 200, 256]
    q = torch.randn(sum(lq), H, dqk, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(sum(lk), H, dqk, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(sum(lk), H, dv, device=DEV, dtype=torch.bfloat16)
    cq = torch.tensor([0, 100, 137, 393], dtype=torch.int32, device=DEV)
    ck = torch.tensor([0, 100, 300, 556], dtype=torch.int32, device=DEV)
    got = ops.varlen_attention(q, k, v, cq, ck, dqk ** -0.5, max_q_len=256)
    want = ops.varlen_attention(q.cpu(), k.cpu(), v.cpu(), cq.cpu(), ck.cpu(), dqk ** -0.5).to(DEV)
    assert cos_diff(got, want) < 3e-4


# ------------------------------------------------------------------ sampling
def test_argmax_and_greedy_sample():
    logits = torch.randn(37, 128256, device=DEV, dtype=torch.bfloat16)
    assert torch.equal(ops.argmax(logits), logits.float().argmax(-1))
    t = torch.zeros(37, device=DEV)
    u = torch.rand(37, device=DEV)
    assert torch.equal(ops.sample(logits, t, None, None, None, u), logits.float().argmax(-1))


def _topk_then_topp_keep(probs, k, p):
    """Upstream's order: top-k, renormalise over the kept tokens, then top-p.  Returns (sorted ids, keep mask by rank,
    renormalised probabilities by rank)."""
    sp, si = probs.sort(-1, descending=True)
    V = probs.shape[-1]
    in_k = torch.arange(V, device=probs.device)[None] < k
    pk = torch.where(in_k, sp, torch.zeros_like(sp))
    pk = pk / pk.sum(-1, keepdim=True)
    keep = in_k & ((pk.cumsum(-1) - pk) < p)
    final = torch.where(keep, pk, torch.zeros_like(pk))
    return si, keep, final / final.sum(-1, keepdim=True)


def test_sample_respects_topk_topp():
    V = 5000
    logits = torch.randn(64, V, device=DEV)
    temp = torch.full((64,), 0.8, device=DEV)
    top_k = torch.full((64,), 50, device=DEV, dtype=torch.int32)
    top_p = torch.full((64,), 0.9, device=DEV)
    si, keep, _ = _topk_then_topp_keep(torch.softmax(logits / 0.8, -1), 50, 0.9)
    for trial in range(8):
        u = torch.rand(64, device=DEV)
        tok = ops.sample(logits, temp, top_k, top_p, None, u)
        rank = (si == tok[:, None]).float().argmax(-1)
        assert bool(keep.gather(1, rank[:, None]).all())


def test_sample_topk_then_topp_distribution():
    """With both cuts active the kept set is the one of the sort-based oracle (top-p over the renormalised top-k
    distribution), and tokens are drawn in proportion inside it."""
    V, n = 64, 16384
    row = torch.randn(1, V, device=DEV)
    logits = row.repeat(n, 1)
    temp = torch.ones(n, device=DEV)
    si, keep, final = _topk_then_topp_keep(torch.softmax(row, -1), 16, 0.8)
    tok = ops.sample(logits, temp, torch.full((n,), 16, device=DEV, dtype=torch.int32),
                     torch.full((n,), 0.8, device=DEV), None, torch.rand(n, device=DEV))
    emp = torch.bincount(tok, minlength=V).float() / n
    want = torch.zeros(V, device=DEV)
    want[si[0]] = final[0]
    assert float(emp[want == 0].sum()) == 0.0
    assert (emp - want).abs().max() < 0.03


def test_sample_distribution_matches():
    V = 50
    logits = torch.randn(1, V, device=DEV).repeat(4096, 1)
    temp = torch.ones(4096, device=DEV)
    u = torch.rand(4096, device=DEV)
    tok = ops.sample(logits, temp, None, None, None, u)
    emp = torch.bincount(tok, minlength=V).float() / 4096
    assert (emp - torch.softmax(logits[0], -1)).abs().max() < 0.04


def test_penalties_and_advance_and_embedding():
    B, V = 5, 1000
    logits = torch.randn(B, V, device=DEV)
    counts = torch.randint(0, 3, (B, V), device=DEV, dtype=torch.int32)
    pm = torch.randint(0, 2, (B, V), device=DEV, dtype=torch.int32)
    rep = torch.full((B,), 1.3, device=DEV)
    pres = torch.full((B,), 0.2, device=DEV)
    freq = torch.full((B,), 0.1, device=DEV)
    want = ops.apply_penalties(logits.cpu().clone(), pm.cpu(), counts.cpu(), rep.cpu(), pres.cpu(), freq.cpu())
    got = ops.apply_penalties(logits.clone(), pm, counts, rep, pres, freq)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)
    table = torch.randn(300, 256, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 300, (40,), device=DEV)
    assert torch.equal(ops.embedding(table, ids), table[ids])
    # advance
    bs, MB = 16, 8
    bt = torch.randint(0, 100, (B, MB), device=DEV, dtype=torch.int32)
    pos = torch.tensor([0, 15, 16, 31, 100], device=DEV)
    ids2 = torch.zeros(B, dtype=torch.int64, device=DEV)
    sl = (pos + 1).to(torch.int32)
    slots = torch.zeros(B, dtype=torch.int64, device=DEV)
    sampled = torch.arange(B, device=DEV) + 7
    ops.advance_step(ids2, pos, sl, slots, sampled, bt, bs, B)
    assert torch.equal(ids2, sampled)
    assert pos.tolist() == [1, 16, 17, 32, 101]
    assert sl.tolist() == [2, 17, 18, 33, 102]
    exp = [int(bt[i, p // bs]) * bs + p % bs for i, p in enumerate([1, 16, 17, 32, 101])]
    assert slots.tolist() == exp


@pytest.mark.parametrize("M", [5, 48, 256, 1000])
def test_gemm_fused_silu_gate_epilogue(M):
    K, I = 1024, 1408
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(2 * I, K, device=DEV, dtype=torch.bfloat16) * 0.05
    got = ops.gemm_silu_mul(a, w)
    want = ops.gemm_silu_mul(a.cpu(), w.cpu()).to(DEV)
    assert got.shape == (M, I)
    assert cos_diff(got, want) < 1e-4
    torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (1024, 1536, 4096), (1000, 1288, 520), (8192, 6144, 4096)])
def test_gemm_cta_pair(M, N, K):
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    want = a.float() @ w.float().t() + bias.float() + res.float()
    got = ops.gemm(a, w, bias, res, force_bn=512)
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2
    assert cos_diff(got, want) < 1e-5


@pytest.mark.parametrize("D", [64, 128])
def test_alibi_bias_in_prefill_and_decode(D):
    """ALiBi slopes: score += slope[h] * (kv position - query position), both attention kernels."""
    torch.manual_seed(9)
    Hq, Hkv, bs = 8, 2, 16
    lens, qlens = [70, 33, 130], [70, 1, 17]          # fresh prefill, decode, chunked prefill
    B = len(lens)
    nblk = [(l + bs - 1) // bs for l in lens]
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    perm = torch.randperm(sum(nblk) + 1)
    o = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[o:o + nblk[b]].int()
        o += nblk[b]
    cache = torch.randn(sum(nblk) + 1, 2, bs, Hkv, D).bfloat16()
    q = torch.randn(sum(qlens), Hq, D).bfloat16()
    slopes = torch.tensor([2.0 ** (-(i + 1)) for i in range(Hq)])
    sl = torch.tensor(lens, dtype=torch.int32)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    want = ref.paged_attention(q.float(), cache.float(), bt, sl, qsl, D ** -0.5, alibi_slopes=slopes)
    plain = ref.paged_attention(q.float(), cache.float(), bt, sl, qsl, D ** -0.5)
    assert (want - plain).abs().max() > 1e-2          # the bias matters in this case
    got_p = ops.paged_attention_prefill(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), qsl.cuda(), D ** -0.5,
                                        max_q_len=max(qlens), alibi_slopes=slopes.cuda())
    torch.testing.assert_close(got_p.float().cpu(), want, rtol=3e-2, atol=3e-2)
    got_d = ops.paged_attention_decode(q.cuda(), cache.cuda(), bt.cuda(), sl.cuda(), D ** -0.5, query_start_loc=qsl.cuda(),
                                       max_q_len=max(qlens), max_seq_len=max(lens), alibi_slopes=slopes.cuda())
    torch.testing.assert_close(got_d.float().cpu(), want, rtol=3e-2, atol=3e-2)
