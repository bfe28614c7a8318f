"""Small fused kernels against their fp32 PyTorch statements (CPU: the wrappers' fallback logic; GPU: the kernels)."""
import pytest
import torch

from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.ops import extra as X
from vllm_metax_b200.ops import reference as ref

gpu = pytest.mark.gpu


def cos_diff(a, b):
    a, b = a.float().flatten().cpu(), b.float().flatten().cpu()
    return 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


def _cos_sin(max_pos, rot, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, rot, 2).float() / rot))
    f = torch.arange(max_pos).float()[:, None] * inv[None]
    return torch.cat([f.cos(), f.sin()], dim=-1).contiguous()


def test_selective_scan_varlen_matches_dense_cpu():
    torch.manual_seed(0)
    d, n, g = 32, 16, 2
    lens = [5, 9]
    A = -torch.rand(d, n)
    us = [torch.randn(1, d, L) for L in lens]
    dts = [torch.rand(1, d, L) for L in lens]
    Bs = [torch.randn(1, g, n, L) for L in lens]
    Cs = [torch.randn(1, g, n, L) for L in lens]
    Dv = torch.randn(d)
    dense = [X.selective_scan_fwd(us[i], dts[i], A, Bs[i], Cs[i], Dv, delta_softplus=True)[0] for i in range(2)]
    qsl = torch.tensor([0, 5, 14], dtype=torch.int32)
    u = torch.cat([x[0] for x in us], -1)
    dt = torch.cat([x[0] for x in dts], -1)
    B = torch.cat([x[0] for x in Bs], -1)
    C = torch.cat([x[0] for x in Cs], -1)
    y, st = X.selective_scan_fwd(u, dt, A, B, C, Dv, delta_softplus=True, query_start_loc=qsl)
    torch.testing.assert_close(y[:, :5], dense[0][0])
    torch.testing.assert_close(y[:, 5:], dense[1][0])
    # chunked: running the second half with the saved state continues the recurrence
    y1, st1 = X.selective_scan_fwd(us[1][:, :, :4], dts[1][:, :, :4], A, Bs[1][..., :4], Cs[1][..., :4], Dv, delta_softplus=True)
    y2, _ = X.selective_scan_fwd(us[1][:, :, 4:], dts[1][:, :, 4:], A, Bs[1][..., 4:], Cs[1][..., 4:], Dv, delta_softplus=True,
                                 ssm_states=st1, has_initial_state=torch.tensor([True]))
    torch.testing.assert_close(torch.cat([y1, y2], -1), dense[1])


def test_fused_qk_norm_rope_cpu_consistency():
    torch.manual_seed(1)
    T, hq, hk, hv, D = 3, 4, 2, 2, 64
    qkv = torch.randn(T, (hq + hk + hv) * D)
    v_before = qkv[:, (hq + hk) * D:].clone()
    cs = _cos_sin(32, D)
    X.fused_qk_norm_rope(qkv, torch.ones(D), torch.ones(D), cs, torch.tensor([0, 3, 7]), hq, hk, hv, D)
    assert torch.equal(qkv[:, (hq + hk) * D:], v_before)
    q0 = qkv[0, :D]                       # position 0: rotation is the identity, rows are unit-RMS
    assert abs(float(q0.pow(2).mean()) - 1.0) < 1e-3


# ----------------------------------------------------------------------------- GPU
@gpu
@pytest.mark.parametrize("M,N,K", [(1, 256, 7168), (7, 2112, 7168), (16, 384, 6144), (32, 128, 3072), (20, 264, 512)])
@pytest.mark.parametrize("f32_out", [False, True])
def test_small_gemm_gpu(M, N, K, f32_out, kernel_status_ok):
    torch.manual_seed(2)
    x = (torch.randn(M, K) * 0.5).bfloat16().cuda()
    w = (torch.randn(N, K) * 0.05).bfloat16().cuda()
    bias = None if f32_out else (torch.randn(N) * 0.1).bfloat16().cuda()
    out = X.small_gemm(x, w, bias, torch.float32 if f32_out else None)
    want = x.float().cpu() @ w.float().cpu().t() + (0 if bias is None else bias.float().cpu())
    assert out.dtype == (torch.float32 if f32_out else torch.bfloat16)
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2 if not f32_out else 2e-3, atol=2e-2 if not f32_out else 2e-3)


@gpu
@pytest.mark.parametrize("D,rot,neox", [(128, 128, True), (128, 64, True), (64, 64, False), (256, 128, True), (128, 128, False)])
def test_fused_qk_norm_rope_gpu(D, rot, neox, kernel_status_ok):
    torch.manual_seed(3)
    T, hq, hk, hv = 37, 8, 2, 2
    qkv = torch.randn(T, (hq + hk + hv) * D).bfloat16()
    qw, kw = (torch.rand(D) + 0.5).bfloat16(), (torch.rand(D) + 0.5).bfloat16()
    cs = _cos_sin(512, rot)
    pos = torch.randint(0, 512, (T,))
    want = X.fused_qk_norm_rope(qkv.float().clone(), qw.float(), kw.float(), cs, pos, hq, hk, hv, D, neox, 1e-6)
    got = X.fused_qk_norm_rope(qkv.cuda(), qw.cuda(), kw.cuda(), cs.cuda(), pos.cuda(), hq, hk, hv, D, neox, 1e-6)
    torch.testing.assert_close(got.float().cpu(), want, rtol=3e-2, atol=3e-2)


@gpu
def test_mla_rope_cache_concat_permute_gpu(kernel_status_ok):
    torch.manual_seed(4)
    T, H, bs, nb = 19, 16, 64, 4
    q_pe = torch.randn(T, H, 64).bfloat16()
    k_pe = torch.randn(T, 64).bfloat16()
    kv_c = torch.randn(T, 512).bfloat16()
    cs = _cos_sin(256, 64)
    pos = torch.randint(0, 256, (T,))
    slots = torch.randperm(nb * bs)[:T]
    cache_cpu = torch.zeros(nb, bs, 576, dtype=torch.bfloat16)
    q_ref, k_ref = q_pe.float().clone(), k_pe.float().clone()
    X.mla_rope_and_cache(q_ref, k_ref, kv_c.float(), cache_cpu.float(), cs, pos, slots)
    cache = torch.zeros(nb, bs, 576, dtype=torch.bfloat16, device="cuda")
    qg, kg = q_pe.cuda(), k_pe.cuda()
    X.mla_rope_and_cache(qg, kg, kv_c.cuda(), cache, cs.cuda(), pos.cuda(), slots.cuda())
    torch.testing.assert_close(qg.float().cpu(), q_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(kg.float().cpu(), k_ref, rtol=2e-2, atol=2e-2)
    flat = cache.reshape(-1, 576).cpu()
    assert torch.equal(flat[slots, :512], kv_c) and torch.equal(flat[slots, 512:], kg.cpu())
    nope = torch.randn(T, H, 512).bfloat16().cuda()
    assert torch.equal(X.concat_mla_q(nope, qg), torch.cat([nope, qg], -1))
    a = torch.randn(9, 256).bfloat16().cuda()
    perm = torch.randperm(256).cuda()
    assert torch.equal(X.permute_cols(a, perm), a[:, perm])


@gpu
@pytest.mark.parametrize("records", [False, True])
def test_gather_mla_cache_gpu(records, kernel_status_ok):
    torch.manual_seed(5)
    nb, bs = 12, 64
    lens = [70, 1, 130]
    kv = torch.randn(nb * bs, 512).bfloat16()
    pe = torch.randn(nb * bs, 64).bfloat16()
    if records:
        cache = ref.pack_ds_mla(kv, pe).reshape(nb, bs, 656)
    else:
        cache = torch.cat([kv, pe], -1).reshape(nb, bs, 576)
    bt = torch.stack([torch.randperm(nb)[:3] for _ in lens]).int()
    cu = torch.tensor([0, 70, 71, 201], dtype=torch.int32)
    want = X.gather_mla_cache(cache, bt, cu, 201, torch.bfloat16)
    got = X.gather_mla_cache(cache.cuda(), bt.cuda(), cu.cuda(), 201, torch.bfloat16)
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=1e-2, atol=1e-2)


@gpu
def test_gather_indexer_k_gpu(kernel_status_ok):
    torch.manual_seed(6)
    nb, bs = 6, 64
    cache = torch.zeros(nb, bs * 132, dtype=torch.uint8)
    k = torch.randn(nb * bs, 128)
    ref.indexer_k_quant_and_cache(k, cache, torch.arange(nb * bs))
    bt = torch.tensor([[3, 1, 5], [0, 2, 4]], dtype=torch.int32)
    cu = torch.tensor([0, 100, 165], dtype=torch.int32)
    wk, ws = X.gather_indexer_k(cache, bt, cu, 165, bs)
    gk, gs = X.gather_indexer_k(cache.cuda(), bt.cuda(), cu.cuda(), 165, bs)
    assert torch.equal(gk.cpu(), wk) and torch.equal(gs.cpu(), ws)


@gpu
@pytest.mark.parametrize("n,g,dtype", [(16, 1, torch.bfloat16), (16, 4, torch.float32), (64, 2, torch.bfloat16), (128, 1, torch.float16)])
def test_selective_scan_gpu(n, g, dtype, kernel_status_ok):
    torch.manual_seed(7)
    d = 64
    lens = [33, 1, 70]
    T = sum(lens)
    qsl = torch.tensor([0, 33, 34, 104], dtype=torch.int32)
    A = -torch.rand(d, n) * 0.5
    u, dt, z = torch.randn(d, T).to(dtype), (torch.rand(d, T) * 0.5).to(dtype), torch.randn(d, T).to(dtype)
    B, C = torch.randn(g, n, T).to(dtype), torch.randn(g, n, T).to(dtype)
    Dv, bias = torch.randn(d), torch.randn(d) * 0.1
    st0 = torch.randn(5, d, n)
    ci = torch.tensor([4, 0, 2], dtype=torch.int32)
    his = torch.tensor([True, False, True])
    want, wst = X.selective_scan_fwd(u.float(), dt.float(), A, B.float(), C.float(), Dv, z.float(), bias, True, st0.clone(), qsl, ci, his)
    got, gst = X.selective_scan_fwd(u.cuda(), dt.cuda(), A.cuda(), B.cuda(), C.cuda(), Dv.cuda(), z.cuda(), bias.cuda(), True,
                                    st0.clone().cuda(), qsl.cuda(), ci.cuda(), his.cuda())
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    assert cos_diff(got, want) < (1e-6 if dtype == torch.float32 else 1e-4)
    torch.testing.assert_close(gst.cpu()[[4, 0, 2]], wst[[4, 0, 2]], rtol=tol, atol=tol)
    assert torch.equal(gst.cpu()[[1, 3]], st0[[1, 3]])


# ----------------------------------------------------------------------------- whole-row norm + RoPE + inserts
def _m3_case(dtype, T=21, hq=6, hk=2, niq=3, bs=16, nb=4, n_insert=18):
    g = torch.Generator().manual_seed(11)
    width = (hq + 2 * hk + niq + 1) * 128
    qkv = torch.randn(T, width, generator=g).to(dtype)
    ws = [(torch.randn(128, generator=g) * 0.1).to(dtype) for _ in range(4)]
    cs = _cos_sin(256, 64)
    pos = torch.randint(0, 256, (T,), generator=g)
    slots = torch.randperm(nb * bs, generator=g)[:n_insert]
    slots[3] = -1
    return qkv, ws, cs, pos, slots, (hq, hk, niq, bs, nb)


def test_qkv_norm_rope_insert_cpu_consistency():
    qkv, ws, cs, pos, slots, (hq, hk, niq, bs, nb) = _m3_case(torch.float32)
    before = qkv.clone()
    kv_cache = torch.zeros(nb, 2, bs, hk, 128)
    idx_cache = torch.zeros(nb * bs, 128)
    q_out, iq_out = X.qkv_norm_rope_insert(qkv, pos, slots, cs, hq, hk, ws[0], ws[1], kv_cache, niq, True, ws[2], ws[3],
                                           idx_cache)
    assert q_out.shape == (21, hq, 128) and iq_out.shape == (21, niq, 128)
    # same math as the in-place q/k op on the leading [q | k | v] part
    part = before[:, : (hq + 2 * hk) * 128].clone()
    X.fused_qk_norm_rope(part, ws[0], ws[1], cs, pos, hq, hk, hk, 128, True, 1e-6, gemma=True)
    torch.testing.assert_close(q_out.reshape(21, -1), part[:, : hq * 128])
    torch.testing.assert_close(qkv[:, hq * 128: (hq + hk) * 128], part[:, hq * 128: (hq + hk) * 128])
    assert torch.equal(qkv[:, (hq + hk) * 128:], before[:, (hq + hk) * 128:])       # v and index parts untouched
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        blk, p = divmod(s, bs)
        torch.testing.assert_close(kv_cache[blk, 0, p].reshape(-1), qkv[t, hq * 128: (hq + hk) * 128])
        torch.testing.assert_close(kv_cache[blk, 1, p].reshape(-1), before[t, (hq + hk) * 128: (hq + 2 * hk) * 128])
    untouched = torch.ones(nb * bs, dtype=torch.bool)
    untouched[slots[slots >= 0]] = False
    assert idx_cache[untouched].abs().max() == 0 and idx_cache[~untouched].abs().min(dim=1).values.max() > 0


@gpu
@pytest.mark.parametrize("fp8_idx", [False, True])
def test_qkv_norm_rope_insert_gpu(fp8_idx, kernel_status_ok):
    qkv, ws, cs, pos, slots, (hq, hk, niq, bs, nb) = _m3_case(torch.bfloat16)
    idt = torch.uint8 if fp8_idx else torch.bfloat16
    kv_ref, idx_ref = torch.zeros(nb, 2, bs, hk, 128), torch.zeros(nb * bs, 128, dtype=torch.uint8 if fp8_idx else torch.float32)
    qkv_ref = qkv.float().clone()
    q_ref, iq_ref = X.qkv_norm_rope_insert(qkv_ref, pos, slots, cs, hq, hk, ws[0].float(), ws[1].float(), kv_ref, niq, True,
                                           ws[2].float(), ws[3].float(), idx_ref, index_fp8=fp8_idx)
    kv = torch.zeros(nb, 2, bs, hk, 128, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(nb * bs, 128, dtype=idt, device="cuda")
    wide = torch.zeros(qkv.shape[0], qkv.shape[1] + 64, dtype=torch.bfloat16, device="cuda")     # padded row pitch
    wide[:, : qkv.shape[1]] = qkv.cuda()
    view = wide[:, : qkv.shape[1]]
    q_out, iq_out = X.qkv_norm_rope_insert(view, pos.cuda(), slots.cuda(), cs.cuda(), hq, hk, ws[0].cuda(), ws[1].cuda(), kv,
                                           niq, True, ws[2].cuda(), ws[3].cuda(), idx, index_fp8=fp8_idx)
    tol = dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(q_out.float().cpu(), q_ref, **tol)
    torch.testing.assert_close(view.float().cpu(), qkv_ref, **tol)
    torch.testing.assert_close(kv.float().cpu(), kv_ref, **tol)

    def f(x):
        return x.view(torch.float8_e4m3fn).float() if fp8_idx else x.float()

    torch.testing.assert_close(f(iq_out.cpu()), f(iq_ref), rtol=0.14 if fp8_idx else 3e-2, atol=3e-2)
    torch.testing.assert_close(f(idx.cpu()), f(idx_ref), rtol=0.14 if fp8_idx else 3e-2, atol=3e-2)
    # dense layer form: no index heads, no cache (profiling run)
    q2, none = X.qkv_norm_rope_insert(qkv[:, : (hq + 2 * hk) * 128].cuda().contiguous(), pos.cuda(), slots.cuda()[:0], cs.cuda(),
                                      hq, hk, ws[0].cuda(), ws[1].cuda())
    assert none is None
    torch.testing.assert_close(q2.float().cpu(), q_ref, **tol)
