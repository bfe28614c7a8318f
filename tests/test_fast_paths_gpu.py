"""Serving-shape fast paths against fp32 PyTorch references: the stream-K skinny GEMM, the two-tile prefill
attention at long contexts and with large score ranges, the register-resident RMSNorm, the vector RoPE+cache path."""
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


# ------------------------------------------------------------------ stream-K GEMM (force_bn = 2000)
@pytest.mark.parametrize("M,N,K", [(256, 6144, 4096), (256, 4096, 14336), (1, 4096, 4096), (7, 768, 4096),
                                   (100, 520, 1024), (129, 3584, 512), (300, 1000, 200), (1000, 1536, 1792),
                                   (16, 256, 64), (256, 28672, 512)])
def test_gemm_streamk_forced(M, N, K):
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    want = a.float() @ w.float().t() + bias.float() + res.float()
    got = ops.gemm(a, w, bias, res, force_bn=2000)
    assert (got.float() - want).abs().max() / want.abs().max() < 1.5e-2
    # partials are added in a fixed order: a second launch gives the same bits, and the counters were reset
    again = ops.gemm(a, w, bias, res, force_bn=2000)
    assert torch.equal(got, again)


def test_gemm_streamk_default_dispatch_and_silu_gate():
    a = torch.randn(256, 4096, device=DEV, dtype=torch.float16)
    w = torch.randn(2048, 4096, device=DEV, dtype=torch.float16) * 0.02
    want = a.float() @ w.float().t()
    assert (ops.gemm(a, w).float() - want).abs().max() / want.abs().max() < 1.5e-2
    for M in (5, 48, 256, 700):
        x = torch.randn(M, 1024, device=DEV, dtype=torch.bfloat16)
        wg = torch.randn(2048, 1024, device=DEV, dtype=torch.bfloat16) * 0.05
        y = x.float() @ wg.float().t()
        want2 = torch.nn.functional.silu(y[:, 0::2].bfloat16().float()) * y[:, 1::2].bfloat16().float()
        got2 = ops.gemm_silu_mul(x, wg)
        assert (got2.float() - want2).abs().max() / want2.abs().max() < 2e-2


def test_gemm_streamk_strided_views():
    base = torch.randn(200, 3 * 1024, device=DEV, dtype=torch.bfloat16)
    a = base[:, 1024:2048]
    w = torch.randn(768, 1024, device=DEV, dtype=torch.bfloat16) * 0.05
    out = torch.zeros(200, 1024, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, w, out=out[:, :768], force_bn=2000)
    want = a.float() @ w.float().t()
    assert (out[:, :768].float() - want).abs().max() / want.abs().max() < 1.5e-2
    assert float(out[:, 768:].abs().max()) == 0.0


# ------------------------------------------------------------------ prefill attention, two query tiles per CTA
def _paged(B, lens, Hkv, D, bs):
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + 1
    cache = torch.randn(total, 2, bs, Hkv, D, device=DEV, dtype=torch.bfloat16)
    perm = torch.randperm(total - 1, device=DEV).to(torch.int32) + 1
    bt = torch.zeros(B, max(nblk), dtype=torch.int32, device=DEV)
    o = 0
    for i, n in enumerate(nblk):
        bt[i, :n] = perm[o:o + n]
        o += n
    return cache, bt


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 8, 64), (16, 16, 128)])
def test_prefill_long_context(Hq, Hkv, D):
    cases = [(1024, 1024), (640, 2048), (33, 1500), (300, 300)]
    lens = [c[1] for c in cases]
    cache, bt = _paged(len(cases), lens, Hkv, D, 128)
    T = sum(c[0] for c in cases)
    q = torch.randn(T, Hq, D, device=DEV, dtype=torch.bfloat16)
    qsl = torch.tensor([0] + list(torch.tensor([c[0] for c in cases]).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    lse = torch.empty(Hq, T, device=DEV)
    got = ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, max_q_len=1024, lse_out=lse)
    want, wlse = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, return_lse=True)
    assert cos_diff(got, want) < 3e-4
    torch.testing.assert_close(got.float(), want.float(), rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(lse, wlse, rtol=2e-2, atol=2e-2)


def test_prefill_row_maximum_grows_late():
    """Keys late in the context score far higher than the early ones, so the lazily tracked row maximum has to
    move (and the TMEM-resident output has to be rescaled) several tiles into the walk."""
    Hq, Hkv, D, bs = 8, 2, 128, 128
    L = 1024
    cache, bt = _paged(1, [L], Hkv, D, bs)
    q = torch.randn(L, Hq, D, device=DEV, dtype=torch.bfloat16)
    # scale up the keys of the later pages: scores there are ~8x larger
    for blk in range(4, 8):
        cache[bt[0, blk].long(), 0] *= 8.0
    qsl = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    sl = torch.tensor([L], dtype=torch.int32, device=DEV)
    got = ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, max_q_len=L)
    want = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5)
    assert cos_diff(got, want) < 5e-4
    torch.testing.assert_close(got.float(), want.float(), rtol=5e-2, atol=5e-2)


def test_varlen_noncausal_and_fp16():
    H, D = 4, 64
    lq, lk = [200, 77], [200, 300]
    q = torch.randn(sum(lq), H, D, device=DEV, dtype=torch.float16)
    k = torch.randn(sum(lk), H, D, device=DEV, dtype=torch.float16)
    v = torch.randn(sum(lk), H, D, device=DEV, dtype=torch.float16)
    cq = torch.tensor([0, 200, 277], dtype=torch.int32, device=DEV)
    ck = torch.tensor([0, 200, 500], dtype=torch.int32, device=DEV)
    got = ops.varlen_attention(q, k, v, cq, ck, D ** -0.5, max_q_len=200, causal=False)
    want = ops.varlen_attention(q.cpu(), k.cpu(), v.cpu(), cq.cpu(), ck.cpu(), D ** -0.5, causal=False).to(DEV)
    assert cos_diff(got, want) < 3e-4


# ------------------------------------------------------------------ norms / rope at serving shapes
@pytest.mark.parametrize("T,H", [(64, 4096), (100, 2048), (40, 1024), (256, 8192)])
def test_rms_norm_register_path(T, H):
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(H, device=DEV, dtype=torch.bfloat16)
    torch.testing.assert_close(ops.rms_norm(x, w, 1e-5), ref.rms_norm(x, w, 1e-5), rtol=2e-2, atol=2e-2)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    wy, wr = ref.fused_add_rms_norm(x, r, w, 1e-5)
    x2, r2 = x.clone(), r.clone()
    ops.fused_add_rms_norm(x2, r2, w, 1e-5)
    torch.testing.assert_close(r2, wr, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(x2, wy, rtol=2e-2, atol=2e-2)


def test_rope_and_cache_vector_path_llama_shape():
    T, Hq, Hk, D, bs, nb = 300, 32, 8, 128, 128, 4
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=DEV, dtype=torch.bfloat16)
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D:(Hq + Hk) * D], qkv[:, (Hq + Hk) * D:]
    pos = torch.randint(0, 2000, (T,), device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[5] = -1
    cos_sin = ref.build_rope_cache(D, 2048, 500000.0).to(DEV)
    cache = torch.zeros(nb, 2, bs, Hk, D, device=DEV, dtype=torch.bfloat16)
    wcache = cache.clone()
    wq, wk = ref.rotary_embedding(pos, q.contiguous(), k.contiguous(), D, cos_sin, True)
    ref.reshape_and_cache(wk.reshape(T, Hk, D), v.reshape(T, Hk, D), wcache, slots, None, 1.0, 1.0)
    ops.rope_and_cache(pos, q, k, v, D, cos_sin, True, cache, slots, None, 1.0, 1.0)
    torch.testing.assert_close(q, wq, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(k, wk, rtol=2e-2, atol=2e-2)
    assert cos_diff(cache.float(), wcache.float()) < 1e-4


# ------------------------------------------------------------------ expert alignment and greedy argmax at serving sizes
@pytest.mark.parametrize("T,topk,E,block,mapped", [(8192, 8, 128, 128, False), (8192, 8, 128, 128, True),
                                                   (256, 8, 256, 128, False), (3, 2, 8, 16, False),
                                                   (1000, 6, 160, 64, True), (4100, 1, 512, 128, False)])
def test_moe_align_matches_stable_sort(T, topk, E, block, mapped):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.randint(0, E, (T, topk), generator=g, dtype=torch.int32)
    emap, local = None, E
    if mapped:
        local = E // 4
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[local: 2 * local] = torch.arange(local, dtype=torch.int32)
    want = ops.moe_align_block_size(ids, block, local, emap, want_inverse=True)
    got = ops.moe_align_block_size(ids.to(DEV), block, local, None if emap is None else emap.to(DEV), want_inverse=True)
    total = int(want[2])
    assert int(got[2]) == total
    assert torch.equal(got[0][:total].cpu(), want[0][:total])
    assert torch.equal(got[1][: total // block].cpu(), want[1][: total // block])
    assert torch.equal(got[3].cpu(), want[3])


@pytest.mark.parametrize("rows,vocab", [(1, 151936), (8, 151936), (37, 128256), (256, 128256), (300, 32000), (5, 1000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax_split_rows(rows, vocab, dtype):
    logits = torch.randn(rows, vocab, device=DEV, dtype=dtype)
    hot = torch.randint(0, vocab, (rows,), device=DEV)
    logits[torch.arange(rows, device=DEV), hot] = 50.0
    assert torch.equal(ops.argmax(logits), hot)
    assert torch.equal(ops.argmax(logits), hot)          # the row tickets were reset
    # ties go to the lowest index; rows that start off a 16-byte boundary take the scalar path
    wide = torch.zeros(rows, vocab + 3, device=DEV, dtype=dtype)
    view = wide[:, 3:]
    view[:, vocab // 2] = 1.0
    view[:, vocab - 1] = 1.0
    assert torch.equal(ops.argmax(view), torch.full((rows,), vocab // 2, device=DEV))
