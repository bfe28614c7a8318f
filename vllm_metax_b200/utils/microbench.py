"""Kernel micro-benchmarks at serving shapes (CUDA events, L2 flushed between iterations).

    python -m vllm_metax_b200.utils.microbench --op all
    python -m vllm_metax_b200.utils.microbench --op gemm --m 8192 --n 6144 --k 4096 --iters 3

Each op reports its median time and the achieved TFLOP/s or GB/s; ``--compare`` adds the
library kernel (cuBLAS) time for GEMMs.  With few ``--iters`` and a single ``--op`` the
command doubles as the small case for an ``ncu`` capture of that kernel.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _custom_ops as ops
from ..ops import reference as ref

DEV = "cuda"


class Timer:
    def __init__(self, iters: int, warmup: int):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]


def paged_cache(B, L, Hkv, D, bs, dtype=torch.bfloat16):
    nblk = (L + bs - 1) // bs
    total = B * nblk + 1
    cache = torch.randn(total, 2, bs, Hkv, D, device=DEV, dtype=torch.float32).to(dtype)
    bt = torch.randperm(B * nblk, device=DEV).to(torch.int32).view(B, nblk)
    return cache, bt


def bench_gemm(t: Timer, M, N, K, compare: bool, force_bn: int = 0) -> dict:
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.02
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ms = t(lambda: ops.gemm(a, w, out=out, force_bn=force_bn))
    r = {"ms": round(ms, 4), "tflops": round(2 * M * N * K / ms / 1e9, 1),
         "gbs": round((M * K + N * K + M * N) * 2 / ms / 1e6, 1)}
    if compare:
        mc = t(lambda: torch.mm(a, w.t(), out=out))
        r["cublas_ms"] = round(mc, 4)
        r["cublas_tflops"] = round(2 * M * N * K / mc / 1e9, 1)
    return r


def bench_prefill(t: Timer, B, L, Hq, Hkv, D, bs, compare: bool = False) -> dict:
    cache, bt = paged_cache(B, L, Hkv, D, bs)
    q = torch.randn(B * L, Hq, D, device=DEV, dtype=torch.bfloat16)
    qsl = torch.arange(B + 1, device=DEV, dtype=torch.int32) * L
    sl = torch.full((B,), L, device=DEV, dtype=torch.int32)
    out = torch.empty_like(q)
    ms = t(lambda: ops.paged_attention_prefill(q, cache, bt, sl, qsl, D ** -0.5, out=out, max_q_len=L))
    res = {"ms": round(ms, 4), "tflops": round(4 * B * L * L / 2 * Hq * D / ms / 1e9, 1)}
    if compare:      # the attention library installed on the box, same problem (contiguous K / V)
        try:
            from flash_attn import flash_attn_varlen_func

            k = torch.randn(B * L, Hkv, D, device=DEV, dtype=torch.bfloat16)
            v = torch.randn_like(k)
            lib = t(lambda: flash_attn_varlen_func(q, k, v, qsl, qsl, L, L, causal=True))
            res["flash_attn_ms"] = round(lib, 4)
        except Exception as e:  # noqa: BLE001
            res["flash_attn_ms"] = f"unavailable: {type(e).__name__}"
    return res


def bench_decode(t: Timer, B, L, Hq, Hkv, D, bs, kv="bf16", compare: bool = False) -> dict:
    cache, bt = paged_cache(B, L, Hkv, D, bs)
    scales = None
    eb = 2
    if kv == "int8":
        cache = (cache.float() * 40).round().clamp(-127, 127).to(torch.int8)
        scales = torch.rand(cache.shape[:-1], device=DEV) * 0.02 + 0.01
        eb = 1
    q = torch.randn(B, Hq, D, device=DEV, dtype=torch.bfloat16)
    sl = torch.full((B,), L, device=DEV, dtype=torch.int32)
    out = torch.empty_like(q)
    ms = t(lambda: ops.paged_attention_decode(q, cache, bt, sl, D ** -0.5, out=out, kv_scales=scales, max_seq_len=L))
    res = {"ms": round(ms, 4), "gbs": round(B * L * Hkv * D * eb * 2 / ms / 1e6, 1)}
    if compare and kv == "bf16":
        try:
            from flash_attn import flash_attn_with_kvcache

            kc, vc = cache[:, 0].contiguous(), cache[:, 1].contiguous()        # [blocks, block_size, Hkv, D]
            lib = t(lambda: flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, cache_seqlens=sl, block_table=bt, causal=True))
            res["flash_attn_ms"] = round(lib, 4)
        except Exception as e:  # noqa: BLE001
            res["flash_attn_ms"] = f"unavailable: {type(e).__name__}"
    return res


def bench_elementwise(t: Timer, T, H, I) -> dict:
    res = {}
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    ms = t(lambda: ops.fused_add_rms_norm(x, r, w, 1e-5))
    res["add_rmsnorm"] = {"ms": round(ms, 4), "gbs": round(T * H * 2 * 4 / ms / 1e6, 1)}
    g = torch.randn(T, 2 * I, device=DEV, dtype=torch.bfloat16)
    o = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ms = t(lambda: ops.silu_and_mul(g, o))
    res["silu_mul"] = {"ms": round(ms, 4), "gbs": round(T * I * 2 * 3 / ms / 1e6, 1)}
    qkv = torch.randn(T, 6144, device=DEV, dtype=torch.bfloat16)
    pos = torch.arange(T, device=DEV) % 1024
    cs = ref.build_rope_cache(128, 2048, 500000.0).to(DEV)
    kvc = torch.zeros(T // 128 + 1, 2, 128, 8, 128, device=DEV, dtype=torch.bfloat16)
    slots = torch.arange(T, device=DEV)
    ms = t(lambda: ops.rope_and_cache(pos, qkv[:, :4096], qkv[:, 4096:5120], qkv[:, 5120:], 128, cs, True, kvc, slots))
    res["rope_cache"] = {"ms": round(ms, 4), "gbs": round((T * 5120 * 2 * 2 + T * 2048 * 2 + T * 2048 * 2) / ms / 1e6, 1)}
    return res


def graph_ms(calls: list, replays: int = 7) -> float:
    """Device time per call of a list of launches replayed from ONE CUDA graph (no host launch gaps: the way a
    decode step runs).  The caller rotates the calls over enough distinct operands to exceed L2."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for c in calls:
            c()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for c in calls:
            c()
    ts = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / len(calls))
    ts.sort()
    return ts[len(ts) // 2]


def bench_skinny(t: Timer) -> dict:
    """Decode-batch GEMMs of Llama-3.1-8B at TP 1 and TP 8 shard sizes: the stream-K CTA-pair kernel (force_bn 2000)
    against the cluster split-K kernel (1004), the plain 128-wide tile kernel (128) and cuBLAS.  Times are per launch
    inside a replayed CUDA graph (how decode steps run), weights rotating through more copies than L2 holds."""
    H, I = 4096, 14336
    res = {}
    for tp in (1, 8):
        shapes = {"qkv": (6144 // tp, H), "o": (H, H // tp), "gate_up": (2 * I // tp, H), "down": (H, I // tp)}
        for M in (32, 256):
            for name, (N, K) in shapes.items():
                # weights rotate over enough copies to exceed L2 (126 MB); one graph replays 4 rounds of them
                R = max(2, min(24, (300 << 20) // (N * K * 2) + 1))
                a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
                ws = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(R)]
                out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
                row = {}
                for label, fb in (("streamk", 2000), ("splitk4", 1004), ("tile128", 128 if M > 64 else -32)):
                    calls = [(lambda w=w, fb=fb: ops.gemm(a, w, out=out, force_bn=fb)) for _ in range(4) for w in ws]
                    row[label + "_ms"] = round(graph_ms(calls), 4)
                calls = [(lambda w=w: torch.mm(a, w.t(), out=out)) for _ in range(4) for w in ws]
                row["cublas_ms"] = round(graph_ms(calls), 4)
                row["weights_gbs_streamk"] = round(N * K * 2 / row["streamk_ms"] / 1e6, 1)
                res[f"tp{tp}_{name}_M{M}_{N}x{K}"] = row
    return res


def bench_decode_layer(tp: int, batch: int = 256, ctx: int = 1100) -> dict:
    """Every launch of one Llama-3.1-8B decoder layer at a decode step of `batch` sequences, at the shard sizes of
    tensor-parallel degree `tp` (row-parallel GEMMs with a local epilogue), each timed inside a replayed CUDA graph
    with operands rotating through more copies than L2 holds.  Shows where a decode step's time goes."""
    H, I, D = 4096, 14336, 128
    hq, hkv = 32 // tp, max(1, 8 // tp)
    bf = torch.bfloat16
    res = {}

    def rot(nbytes):
        return max(2, min(16, (300 << 20) // max(1, nbytes) + 1))

    def gemm_row(name, N, K, silu=False):
        R = rot(N * K * 2)
        a = torch.randn(batch, K, device=DEV, dtype=bf)
        ws = [torch.randn(N, K, device=DEV, dtype=bf) * 0.02 for _ in range(R)]
        if silu:
            calls = [(lambda w=w: ops.gemm_silu_mul(a, w)) for _ in range(3) for w in ws]
        else:
            out = torch.empty(batch, N, device=DEV, dtype=bf)
            calls = [(lambda w=w: ops.gemm(a, w, out=out)) for _ in range(3) for w in ws]
        ours = graph_ms(calls)
        out2 = torch.empty(batch, N, device=DEV, dtype=bf)
        lib = graph_ms([(lambda w=w: torch.mm(a, w.t(), out=out2)) for _ in range(3) for w in ws])
        res[name] = {"ms": round(ours, 4), "cublas_ms": round(lib, 4), "weights_gbs": round(N * K * 2 / ours / 1e6, 1)}

    gemm_row("qkv_gemm", (hq + 2 * hkv) * D, H)
    gemm_row("o_gemm", H, hq * D)
    gemm_row("gate_up_silu_gemm", 2 * I // tp, H, silu=True)
    gemm_row("down_gemm", H, I // tp)
    # norm (+ residual)
    x = torch.randn(batch, H, device=DEV, dtype=bf)
    r = torch.randn_like(x)
    w = torch.ones(H, device=DEV, dtype=bf)
    res["add_rmsnorm"] = {"ms": round(graph_ms([lambda: ops.fused_add_rms_norm(x, r, w, 1e-5)] * 20), 4)}
    # rope + cache write
    qkv = torch.randn(batch, (hq + 2 * hkv) * D, device=DEV, dtype=bf)
    pos = torch.full((batch,), ctx, device=DEV)
    cs = ref.build_rope_cache(D, 2048, 500000.0).to(DEV)
    nblk = (ctx + 127) // 128
    caches = [torch.randn(batch * nblk + 1, 2, 128, hkv, D, device=DEV, dtype=bf) for _ in range(rot(batch * nblk * 2 * 128 * hkv * D * 2))]
    slots = torch.arange(batch, device=DEV) * nblk * 128 + ctx - 1
    q_, k_, v_ = qkv[:, :hq * D], qkv[:, hq * D:(hq + hkv) * D], qkv[:, (hq + hkv) * D:]
    res["rope_cache"] = {"ms": round(graph_ms([(lambda c=c: ops.rope_and_cache(pos, q_, k_, v_, D, cs, True, c, slots))
                                               for _ in range(5) for c in caches]), 4)}
    # decode attention
    bt = torch.arange(batch * nblk, device=DEV, dtype=torch.int32).view(batch, nblk)
    sl = torch.full((batch,), ctx, device=DEV, dtype=torch.int32)
    qd = torch.randn(batch, hq, D, device=DEV, dtype=bf)
    od = torch.empty_like(qd)
    att = graph_ms([(lambda c=c: ops.paged_attention_decode(qd, c, bt, sl, D ** -0.5, out=od, max_seq_len=ctx))
                    for _ in range(3) for c in caches])
    res["attn_decode"] = {"ms": round(att, 4), "kv_gbs": round(batch * ctx * hkv * D * 2 * 2 / att / 1e6, 1)}
    res["layer_total_ms"] = round(sum(v["ms"] for v in res.values()) + res["add_rmsnorm"]["ms"], 4)
    return res


def bench_configs(t: Timer) -> dict:
    """Kernels that carry the MoE / MLA / long-context serving configurations, at per-rank shapes of an 8-way
    expert- / tensor-parallel deployment (and the unsharded shape where it fits): grouped expert GEMMs in bf16 and
    block-scaled fp8, absorbed MLA decode (dense and sparse, bf16 rows and 656-byte fp8 records), the sparse-attention
    indexer (logits + top-k), paged decode over an int8 cache at 32 k tokens of context."""
    res = {}
    bf = torch.bfloat16
    # ---- grouped expert GEMMs: (label, local experts, hidden, expert FFN), 8192 routed pairs per rank
    for label, E, H, I in (("qwen3_30b_ep8", 16, 2048, 768), ("dsv3_ep8", 32, 7168, 2048)):
        pairs = 8192
        ids = torch.randint(0, E, (pairs, 1), device=DEV, dtype=torch.int32)
        sorted_ids, block_expert, total, _ = ops.moe_align_block_size(ids, 128, E, None, want_inverse=True)
        R = sorted_ids.shape[0]
        a = torch.randn(R, H, device=DEV, dtype=bf)
        w13 = torch.randn(E, 2 * I, H, device=DEV, dtype=bf) * 0.02
        w2 = torch.randn(E, H, I, device=DEV, dtype=bf) * 0.02
        h = torch.randn(R, I, device=DEV, dtype=bf)
        ms1 = t(lambda: ops.gemm_grouped(a, w13, block_expert, total, epi=1))
        ms2 = t(lambda: ops.gemm_grouped(h, w2, block_expert, total, epi=0))
        res[f"grouped_bf16_{label}_w13"] = {"ms": round(ms1, 4), "tflops": round(2 * pairs * 2 * I * H / ms1 / 1e9, 1)}
        res[f"grouped_bf16_{label}_w2"] = {"ms": round(ms2, 4), "tflops": round(2 * pairs * I * H / ms2 / 1e9, 1)}
        aq, a_s = ops.per_token_group_quant_fp8(a, 128)
        w13q = w13.to(torch.float8_e4m3fn)
        ws13 = torch.ones(E, 2 * I // 128, H // 128, device=DEV, dtype=torch.float32)
        ms3 = t(lambda: ops.fp8_block_scaled_mm(aq, a_s, w13q, ws13, block_expert=block_expert, total_padded=total))
        res[f"grouped_fp8_blockscale_{label}_w13"] = {"ms": round(ms3, 4),
                                                      "tflops": round(2 * pairs * 2 * I * H / ms3 / 1e9, 1)}
        del a, w13, w2, h, aq, w13q
    # ---- routing: 8192 tokens, 256 experts, sigmoid grouped top-8 (DeepSeek) and 128 experts softmax top-8 (Qwen3)
    g256 = torch.randn(8192, 256, device=DEV, dtype=torch.float32)
    bias = torch.zeros(256, device=DEV)
    res["grouped_topk_8192x256"] = {"ms": round(t(lambda: ops.grouped_topk(g256, 8, True, 8, 4, "sigmoid", bias, 2.5)), 4)}
    g128 = torch.randn(8192, 128, device=DEV, dtype=torch.float32)
    res["topk_softmax_8192x128"] = {"ms": round(t(lambda: ops.topk_gating(g128, 8, True, "softmax")), 4)}
    # ---- absorbed MLA decode: batch 128 x 8192 tokens of context, 16 heads (TP 8) and 128 heads
    B, L, bs = 128, 8192, 64
    nblk = L // bs
    bt = torch.arange(B * nblk, device=DEV, dtype=torch.int32).view(B, nblk)
    sl = torch.full((B,), L, device=DEV, dtype=torch.int32)
    cache_bf = torch.randn(B * nblk, bs, 576, device=DEV, dtype=bf)
    cache_f8 = torch.randint(0, 120, (B * nblk, bs, 656), device=DEV, dtype=torch.uint8)
    cache_f8[..., 512:528] = torch.tensor([0, 0, 128, 60] * 4, device=DEV, dtype=torch.uint8)   # scales = 2^-7 (f32)
    for H in (16, 128):
        q = torch.randn(B, H, 576, device=DEV, dtype=bf) * 0.1
        for name, cache, rec in (("bf16", cache_bf, 1152), ("fp8_records", cache_f8, 656)):
            ms = t(lambda: ops.mla_decode(q, cache, bt, sl, 0.07, max_seq_len=L))
            res[f"mla_decode_{name}_h{H}_b{B}x{L}"] = {"ms": round(ms, 4), "cache_gbs": round(B * L * rec / ms / 1e6, 1),
                                                       "tflops": round(2 * B * H * L * (576 + 512) / ms / 1e9, 1)}
        # sparse (top-k 2048 positions per token)
        topk = torch.stack([torch.randperm(L, device=DEV)[:2048] for _ in range(4)]).to(torch.int32).repeat(B // 4, 1)
        ms = t(lambda: ops.mla_decode(q, cache_f8, bt, sl, 0.07, topk_indices=topk, max_seq_len=L))
        res[f"mla_sparse_decode_fp8_h{H}_b{B}_top2048"] = {"ms": round(ms, 4),
                                                            "cache_gbs": round(B * 2048 * 656 / ms / 1e6, 1)}
    # sparse prefill: 1024 new tokens of one request with 8192 tokens of context, 16 heads
    qp = torch.randn(1024, 16, 576, device=DEV, dtype=bf) * 0.1
    qsl = torch.tensor([0, 1024], device=DEV, dtype=torch.int32)
    topk_p = torch.stack([torch.randperm(L, device=DEV)[:2048] for _ in range(8)]).to(torch.int32).repeat(128, 1)
    ms = t(lambda: ops.mla_decode(qp, cache_f8, bt[:1], sl[:1], 0.07, query_start_loc=qsl, topk_indices=topk_p,
                                  max_seq_len=L))
    res["mla_sparse_prefill_fp8_h16_1024tok_top2048"] = {"ms": round(ms, 4),
                                                          "tflops": round(2 * 1024 * 16 * 2048 * 1088 / ms / 1e9, 1)}
    del cache_bf, cache_f8
    # ---- indexer: 64 heads x 128, fp8 keys (132 bytes per token), logits + top-2048
    for Lk, T in ((8192, 1024), (32768, 256)):
        nb = Lk // bs
        idx_cache = torch.randint(0, 100, (nb, bs * 132), device=DEV, dtype=torch.uint8)
        idx_cache.view(nb, bs * 132)[:, bs * 128:] = torch.tensor([0, 0, 128, 60], device=DEV, dtype=torch.uint8).repeat(bs)
        qi = (torch.randn(T, 64, 128, device=DEV) * 0.5).to(torch.float8_e4m3fn)
        wts = torch.rand(T, 64, device=DEV)
        bti = torch.arange(nb, device=DEV, dtype=torch.int32).view(1, nb)
        sli = torch.tensor([Lk], device=DEV, dtype=torch.int32)
        qsli = torch.tensor([0, T], device=DEV, dtype=torch.int32)
        ms = t(lambda: ops.indexer_topk(qi, wts, idx_cache, bti, sli, qsli, 2048, bs, max_seq_len=Lk))
        res[f"indexer_logits_topk_T{T}_L{Lk}"] = {"ms": round(ms, 4),
                                                  "tflops": round(2 * T * 64 * Lk * 128 / ms / 1e9, 1)}
        # the two halves on their own, and the mma.sync logits kernel the tcgen05 one replaces
        lg = torch.empty(T, Lk, device=DEV, dtype=torch.float32)
        for name, impl in (("tcgen05", 2), ("mma_sync", 1)):
            ms = t(lambda: torch.ops.b200.indexer_logits(lg, qi, wts, idx_cache, bti, sli, qsli, bs, Lk, False, 0, impl))
            res[f"indexer_logits_only_{name}_T{T}_L{Lk}"] = {"ms": round(ms, 4),
                                                             "tflops": round(2 * T * 64 * Lk * 128 / ms / 1e9, 1)}
        out_k = torch.empty(T, 2048, device=DEV, dtype=torch.int32)
        ms = t(lambda: torch.ops.b200.topk_per_row(out_k, lg, None, Lk))
        res[f"topk_per_row_2048_T{T}_L{Lk}"] = {"ms": round(ms, 4), "gbs": round(T * Lk * 4 / ms / 1e6, 1)}
    # decode: 128 requests x 1 token over 32768 cached keys each
    nb = 128 * (32768 // bs)
    idx_cache = torch.randint(0, 100, (nb, bs * 132), device=DEV, dtype=torch.uint8)
    idx_cache.view(nb, bs * 132)[:, bs * 128:] = torch.tensor([0, 0, 128, 60], device=DEV, dtype=torch.uint8).repeat(bs)
    qi = (torch.randn(128, 64, 128, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    wts = torch.rand(128, 64, device=DEV)
    bti = torch.arange(nb, device=DEV, dtype=torch.int32).view(128, -1)
    sli = torch.full((128,), 32768, device=DEV, dtype=torch.int32)
    qsli = torch.arange(129, device=DEV, dtype=torch.int32)
    lg = torch.empty(128, 32768, device=DEV, dtype=torch.float32)
    for name, impl in (("tcgen05", 2), ("mma_sync", 1)):
        ms = t(lambda: torch.ops.b200.indexer_logits(lg, qi, wts, idx_cache, bti, sli, qsli, bs, 32768, False, 1, impl))
        res[f"indexer_logits_decode_{name}_b128_L32768"] = {"ms": round(ms, 4),
                                                            "key_gbs": round(128 * 32768 * 132 / ms / 1e6, 1)}
    del idx_cache
    # ---- paged decode over an int8 cache: 32 sequences x 32768 tokens, 8 q / 1 kv head (TP 8) and 64 / 8
    for Hq, Hkv in ((8, 1), (64, 8)):
        res[f"attn_decode_int8kv_32x32768_h{Hq}"] = bench_decode(t, 32, 32768, Hq, Hkv, 128, 128, "int8")
        res[f"attn_decode_bf16kv_32x32768_h{Hq}"] = bench_decode(t, 32, 32768, Hq, Hkv, 128, 128, "bf16")
    return res


def bench_quant(t, M: int, N: int, K: int) -> dict:
    """Quantised GEMMs at one shape (TFLOP/s over 2 M N K) and the TurboQuant decode kernel (bytes of compressed
    cache streamed per second)."""
    from ..ops import turboquant as tq
    from ..quantization import wna16 as W

    res = {}
    flops = 2.0 * M * N * K
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    # fp8, 1x128 activation scales and 128x128 weight scales
    aq, a_s = ops.per_token_group_quant_fp8(x, 128)
    wq = w.to(torch.float8_e4m3fn)
    w_s = torch.ones(N // 128, K // 128, device=DEV, dtype=torch.float32)
    ms = t(lambda: ops.fp8_block_scaled_mm(aq, a_s, wq, w_s))
    res["fp8_blockscale"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}
    # W8A8 int8, per-token / per-channel scales
    a8 = torch.randint(-127, 127, (M, K), device=DEV, dtype=torch.int8)
    w8 = torch.randint(-127, 127, (N, K), device=DEV, dtype=torch.int8)
    sa = torch.rand(M, device=DEV) * 0.01
    sw = torch.rand(N, device=DEV) * 0.01
    ms = t(lambda: ops.scaled_mm(a8, w8, sa, sw))
    res["w8a8_int8"] = {"ms": round(ms, 4), "tops": round(flops / ms / 1e9, 1)}
    ms = t(lambda: ops.scaled_mm(aq.view(torch.float8_e4m3fn), wq, sa, sw))
    res["w8a8_fp8"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}
    # W4A16 (group 128, symmetric): a weight stream at small M
    qv, sg, _ = W.quantize_weight(w.float().cpu(), 4, 128, sym=True)
    qc, sc, zc = (v.to(DEV) for v in W.canonical_from_values(qv, sg, None, 4, torch.bfloat16))
    ms = t(lambda: ops.wna16_gemm(x, qc, sc, zc, 4, 128))
    res["w4a16"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                    "weight_gbs": round(N * K / 2 / ms / 1e6, 1)}
    # TurboQuant decode: 256 sequences x 1100 tokens, 32 / 8 heads
    fmt = tq.TqFormat.from_name("turboquant_4bit_nc")
    B, L, bs = 256, 1100, 128
    nb = B * ((L + bs - 1) // bs)
    cache = torch.randint(0, 255, (nb, bs, 8, fmt.slot_bytes), device=DEV, dtype=torch.uint8)
    cache[..., fmt.k_bytes + fmt.v_bytes:] = 0          # finite norms / scales (fp16 zero)
    bt = torch.arange(nb, device=DEV, dtype=torch.int32).view(B, -1)
    sl = torch.full((B,), L, device=DEV, dtype=torch.int32)
    qd = torch.randn(B, 32, 128, device=DEV, dtype=torch.bfloat16)
    ms = t(lambda: tq.decode_attention(qd, cache, bt, sl, 0.088, fmt))
    res["turboquant_decode_256x1100"] = {"ms": round(ms, 4), "gbs": round(B * L * 8 * fmt.slot_bytes / ms / 1e6, 1)}
    return res


def bench_linear_attention(t: Timer) -> dict:
    """Qwen3-Next linear-attention layer shapes (16 k heads, 32 v heads of 128; convolution over 8192 channels, width 4):
    one prefill chunk of 8192 tokens in 8 sequences and a decode step of 256 sequences."""
    from ..ops import gdn

    Hk, Hv, D, K = 16, 32, 128, 4
    C = 2 * Hk * D + Hv * D
    out = {}
    for name, lens in (("prefill_8x1024", [1024] * 8), ("decode_256", [1] * 256)):
        T, B = sum(lens), len(lens)
        qsl = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
        idx = torch.arange(B, dtype=torch.int32, device=DEV)
        has = torch.ones(B, dtype=torch.int32, device=DEV)
        x = torch.randn(T, C, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(C, K, device=DEV, dtype=torch.bfloat16) * 0.3
        cstate = torch.zeros(B, K - 1, C, device=DEV, dtype=torch.bfloat16)
        ms = t(lambda: gdn.causal_conv1d(x, w, None, cstate, qsl, idx, has))
        byt = 2 * T * C * 2 + 2 * B * (K - 1) * C * 2
        out[f"causal_conv1d_{name}"] = {"ms": round(ms, 4), "gbs": round(byt / ms / 1e6, 1)}
        q = torch.randn(T, Hk, D, device=DEV, dtype=torch.bfloat16)
        k = torch.randn(T, Hk, D, device=DEV, dtype=torch.bfloat16)
        v = torch.randn(T, Hv, D, device=DEV, dtype=torch.bfloat16)
        g = -torch.rand(T, Hv, device=DEV) * 0.3
        beta = torch.rand(T, Hv, device=DEV)
        state = torch.zeros(B, Hv, D, D, device=DEV, dtype=torch.float32)
        ms = t(lambda: gdn.gated_delta_rule(q, k, v, g, beta, qsl, state, idx, has))
        byt = 2 * B * Hv * D * D * 4 + T * (2 * Hk + 2 * Hv) * D * 2
        # per token and v head: decay (D*D), S^T k (2 D*D), rank-1 update (2 D*D), S^T q (2 D*D)
        out[f"gated_delta_rule_{name}"] = {"ms": round(ms, 4), "gbs": round(byt / ms / 1e6, 1),
                                            "gflops": round(7 * T * Hv * D * D / ms / 1e6, 1)}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "gemm", "prefill", "decode", "elementwise", "quant", "linear_attention", "skinny", "decode_layer", "configs", "indexer", "mla"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--force-bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--seq", type=int, default=1100)
    ap.add_argument("--kv", default="bf16")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--compare", action="store_true")
    a = ap.parse_args()
    ops.load_native()
    t = Timer(a.iters, a.warmup)
    res = {}
    H, I, V = 4096, 14336, 128256
    if a.op == "gemm":
        res[f"gemm_{a.m}x{a.n}x{a.k}"] = bench_gemm(t, a.m, a.n, a.k, a.compare, a.force_bn)
    if a.op == "all":
        for M in (8192, 256):
            for name, (N, K) in {"qkv": (6144, H), "o": (H, H), "gate_up": (2 * I, H), "down": (H, I),
                                 "lm_head": (V, H)}.items():
                if name == "lm_head" and M > 256:
                    continue
                res[f"gemm_{name}_M{M}"] = bench_gemm(t, M, N, K, True)
    if a.op == "quant":
        res[f"quant_{a.m}x{a.n}x{a.k}"] = bench_quant(t, a.m, a.n, a.k)
    if a.op in ("all", "prefill"):
        res["attn_prefill_8x1024"] = bench_prefill(t, 8, 1024, 32, 8, 128, 128, a.compare)
    if a.op in ("all", "decode"):
        res[f"attn_decode_{a.batch}x{a.seq}_{a.kv}"] = bench_decode(t, a.batch, a.seq, 32, 8, 128, 128, a.kv, a.compare)
    if a.op == "linear_attention":
        res.update(bench_linear_attention(t))
    if a.op == "skinny":
        res.update(bench_skinny(t))
    if a.op == "configs":
        res.update(bench_configs(t))
    if a.op == "mla":            # absorbed MLA decode, --batch requests x --seq cached tokens, bf16 cache: both kernels
        B, L, bs = a.batch, a.seq, 64
        nblk = (L + bs - 1) // bs
        bt = torch.arange(B * nblk, device=DEV, dtype=torch.int32).view(B, nblk)
        sl = torch.full((B,), L, device=DEV, dtype=torch.int32)
        cache = torch.randn(B * nblk, bs, 576, device=DEV, dtype=torch.bfloat16)
        for Hh in (128, 64, 16):
            q = torch.randn(B, Hh, 576, device=DEV, dtype=torch.bfloat16) * 0.1
            row = {}
            for name, impl in (("mma_sync", 1), ("tcgen05", 2)):
                ms = t(lambda: ops.mla_decode(q, cache, bt, sl, 0.07, max_seq_len=L, impl=impl))
                row[name] = {"ms": round(ms, 4), "cache_gbs": round(B * L * 1152 / ms / 1e6, 1),
                             "tflops": round(2 * B * Hh * L * (576 + 512) / ms / 1e9, 1)}
            o1 = ops.mla_decode(q, cache, bt, sl, 0.07, max_seq_len=L, impl=1).float()
            o2 = ops.mla_decode(q, cache, bt, sl, 0.07, max_seq_len=L, impl=2).float()
            row["max_abs_diff"] = float((o1 - o2).abs().max())
            res[f"mla_decode_bf16_h{Hh}_b{B}x{L}"] = row
    if a.op == "indexer":        # --m query tokens of one request against --n cached keys (fp8, 64 heads): logits only
        T, Lk, bs = a.m, a.n, 64
        nb = Lk // bs
        idx_cache = torch.randint(0, 100, (nb, bs * 132), device=DEV, dtype=torch.uint8)
        idx_cache.view(nb, bs * 132)[:, bs * 128:] = torch.tensor([0, 0, 128, 60], device=DEV, dtype=torch.uint8).repeat(bs)
        qi = (torch.randn(T, 64, 128, device=DEV) * 0.5).to(torch.float8_e4m3fn)
        wts = torch.rand(T, 64, device=DEV)
        bti = torch.arange(nb, device=DEV, dtype=torch.int32).view(1, nb)
        sli = torch.tensor([Lk], device=DEV, dtype=torch.int32)
        qsli = torch.tensor([0, T], device=DEV, dtype=torch.int32)
        lg = torch.empty(T, Lk, device=DEV, dtype=torch.float32)
        ms = t(lambda: torch.ops.b200.indexer_logits(lg, qi, wts, idx_cache, bti, sli, qsli, bs, Lk, False, 0, 2))
        res[f"indexer_logits_tcgen05_T{T}_L{Lk}"] = {"ms": round(ms, 4), "tflops": round(2 * T * 64 * Lk * 128 / ms / 1e9, 1)}
    if a.op == "decode_layer":
        for tp in (1, 8):
            res[f"decode_layer_tp{tp}_b{a.batch}"] = bench_decode_layer(tp, a.batch, a.seq)
    if a.op in ("all", "elementwise"):
        for T in (8192, 256):
            for k, v in bench_elementwise(t, T, H, I).items():
                res[f"{k}_T{T}"] = v
    torch.cuda.synchronize()
    ops.check_kernel_status(0)
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
