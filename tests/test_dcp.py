"""Decode context parallelism on CPU ranks (Gloo): interleaved KV shards + LSE-corrected combine must reproduce
full attention exactly (reference: cp_lse_ag_out_rs in vllm_metax/v1/attention/backends/flash_attn.py:1577-1582)."""
import os
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _attend(q, k, v, scale):
    """q [H, D], k/v [L, Hkv, D] -> out [H, D], lse [H] (GQA; an empty shard gives zeros and -inf)."""
    H, Hkv = q.shape[0], k.shape[1]
    if k.shape[0] == 0:
        return torch.zeros(H, v.shape[-1]), torch.full((H,), float("-inf"))
    kk = k.repeat_interleave(H // Hkv, 1)
    vv = v.repeat_interleave(H // Hkv, 1)
    s = torch.einsum("hd,lhd->hl", q, kk) * scale
    lse = torch.logsumexp(s, -1)
    return torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vv), lse


def test_local_views():
    from vllm_metax_b200.parallel import dcp

    sl = torch.tensor([0, 1, 2, 5, 8])
    assert dcp.local_seq_lens(sl, 2, 0).tolist() == [0, 1, 1, 3, 4]
    assert dcp.local_seq_lens(sl, 2, 1).tolist() == [0, 0, 1, 2, 4]
    assert sum(dcp.local_seq_lens(sl, 4, r) for r in range(4)).tolist() == sl.tolist()
    pos = torch.tensor([4, 5, 6, 7])
    slots = torch.tensor([100, 101, 102, 103])
    assert dcp.local_slot_mapping(slots, pos, 2, 1).tolist() == [-1, 101, -1, 103]
    k = torch.arange(10)
    assert dcp.shard_kv_interleaved(k, 4, 1).tolist() == [1, 5, 9]
    assert dcp.shard_kv_interleaved(k[3:], 4, 1, start=3).tolist() == [5, 9]


def _worker(rank, world, port, q_out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from vllm_metax_b200.parallel import dcp
    from vllm_metax_b200.parallel import state as ps

    ps.init_distributed(tensor_parallel_size=world, decode_context_parallel_size=world, device="cpu")
    g = ps.get_dcp_group()
    assert g.world_size == world
    gen = torch.Generator().manual_seed(0)                  # same tensors on every rank
    H, Hkv, D, scale = 8, 2, 16, 0.25
    hl = H // world
    lens = [1, 2, 7, 64]                                    # 1 and 2: some shards are empty
    q_all = torch.randn(len(lens), H, D, generator=gen)
    ks = [torch.randn(L, Hkv, D, generator=gen) for L in lens]
    vs = [torch.randn(L, Hkv, D, generator=gen) for L in lens]
    want = torch.stack([_attend(q_all[b], ks[b], vs[b], scale)[0] for b in range(len(lens))])
    want_lse = torch.stack([_attend(q_all[b], ks[b], vs[b], scale)[1] for b in range(len(lens))])

    def attend_local(qa):
        outs, lses = zip(*[_attend(qa[b], dcp.shard_kv_interleaved(ks[b], world, rank),
                                   dcp.shard_kv_interleaved(vs[b], world, rank), scale) for b in range(len(lens))])
        return torch.stack(outs), torch.stack(lses)

    q_local = q_all[:, rank * hl:(rank + 1) * hl]
    got, lse = dcp.decode_attention(q_local, attend_local, g, return_lse=True)
    torch.testing.assert_close(got, want[:, rank * hl:(rank + 1) * hl], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lse, want_lse[:, rank * hl:(rank + 1) * hl], rtol=1e-5, atol=1e-5)
    if rank == 0:
        q_out.put("ok")
    ps.destroy()


def test_dcp_decode_matches_full_attention():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 90
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=120) == "ok"
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0


# ------------------------------------------------------------------ MLA (dense and sparse) under DCP, op level
def _mla_step(world, rank):
    """One mixed step (a decode at position 37, a 5-token chunk at positions 20..24, a decode at position 0) through
    ``MLAAttention`` and the sparse indexer: on the whole cache (returned as ``want``) and on this rank's interleaved
    shard with the group's collectives (``got``: this rank's heads)."""
    from vllm_metax_b200 import _custom_ops as ops
    from vllm_metax_b200.attention.metadata import AttentionMetadata, ForwardContext, set_forward_context
    from vllm_metax_b200.layers.mla import MLAAttention, sparse_attn_indexer

    gen = torch.Generator().manual_seed(3)
    H, nope, rope, vh, lora, Hi, topk = 4, 32, 64, 32, 512, 4, 6
    hl = H // world
    scale = (nope + rope) ** -0.5
    kv_b = torch.randn(H * (nope + vh), lora, generator=gen) * 0.05
    full = MLAAttention(H, scale, nope, rope, vh, lora, 0, dtype=torch.float32)
    full.set_kv_b(kv_b)
    mine = MLAAttention(hl, scale, nope, rope, vh, lora, 0, dtype=torch.float32)
    mine.set_kv_b(kv_b.view(H, nope + vh, lora)[rank * hl:(rank + 1) * hl].reshape(-1, lora))
    starts, news = [37, 0, 20], [1, 1, 5]
    blocks = [[3, 1, 5], [2], [4, 0]]                      # scheduler blocks of 16 tokens = 8 local slots x 2 ranks
    vbs, bs = 16, 16 // world
    ctx_c = [torch.randn(s, lora, generator=gen) for s in starts]
    ctx_pe = [torch.randn(s, rope, generator=gen) for s in starts]
    ctx_ik = [torch.randn(s, 128, generator=gen) for s in starts]
    T = sum(news)
    q = torch.randn(T, H, nope + rope, generator=gen)
    kv_c, k_pe = torch.randn(T, lora, generator=gen), torch.randn(T, rope, generator=gen)
    iq = torch.randn(T, Hi, 128, generator=gen).to(torch.float8_e4m3fn)
    iw = torch.rand(T, Hi, generator=gen)
    ik = torch.randn(T, 128, generator=gen)

    def slots(req, pos, d, r, b):
        blk = torch.tensor(blocks[req])
        s = blk[pos // vbs] * b + (pos % vbs) // d
        return torch.where(pos % d == r, s, torch.full_like(s, -1))

    def run(d, r, attn, sparse):
        b = vbs // d
        cache = torch.zeros(8, b, 576)
        icache = torch.zeros(8, b * 132, dtype=torch.uint8)
        for i, s in enumerate(starts):
            if s:
                sm = slots(i, torch.arange(s), d, r, b)
                ops.concat_and_cache_mla(ctx_c[i], ctx_pe[i], cache, sm)
                ops.indexer_k_quant_and_cache(ctx_ik[i], icache, sm, b)
        pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, news)])
        req = torch.cat([torch.full((n,), i) for i, n in enumerate(news)])
        sm = torch.cat([slots(i, torch.arange(s, s + n), d, r, b) for i, (s, n) in enumerate(zip(starts, news))])
        qsl = torch.tensor([0, 1, 2, 7], dtype=torch.int32)
        seq = torch.tensor([(s + n - r + d - 1) // d for s, n in zip(starts, news)], dtype=torch.int32)
        bt = torch.zeros(3, 3, dtype=torch.int32)
        for i, bl in enumerate(blocks):
            bt[i, : len(bl)] = torch.tensor(bl)
        md = AttentionMetadata(num_tokens=T, num_reqs=3, num_decodes=2, num_decode_tokens=2, query_start_loc=qsl,
                               seq_lens=seq, block_table=bt, slot_mapping=sm, max_query_len=5, max_seq_len=38,
                               block_size=b, prefill_query_start_loc=torch.tensor([0, 5], dtype=torch.int32),
                               max_prefill_query_len=5)
        md.extra["prefill_no_context"] = False
        if d > 1:
            md.extra["dcp_ctx_lens"] = torch.zeros(3, dtype=torch.int32)
            md.extra["dcp_any_context"] = True
            md.extra["dcp_vis_lens"] = ((pos - r + d) // d).to(torch.int32)
            md.extra["dcp_token_req"] = req
        heads = slice(r * attn.num_heads, (r + 1) * attn.num_heads) if d > 1 else slice(None)
        with set_forward_context(ForwardContext(attn_metadata=md, kv_caches=[{"mla": cache}])):
            idx = sparse_attn_indexer(iq, iw, ik, icache, topk, b) if sparse else None
            out = attn(q[:, heads].contiguous(), kv_c, k_pe, None, idx)
        return out, idx

    res = {}
    for sparse in (False, True):
        want, want_idx = run(1, 0, full, sparse)
        got, got_idx = run(world, rank, mine, sparse)
        res[sparse] = (want.view(T, H, vh)[:, rank * hl:(rank + 1) * hl].reshape(T, -1), got, want_idx, got_idx)
    return res


def _mla_worker(rank, world, port, q_out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from vllm_metax_b200.parallel import state as ps

    ps.init_distributed(tensor_parallel_size=world, decode_context_parallel_size=world, device="cpu")
    res = _mla_step(world, rank)
    for sparse, (want, got, want_idx, got_idx) in res.items():
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
        if sparse:
            assert torch.equal(want_idx.sort(1).values, got_idx.sort(1).values), (want_idx, got_idx)
    if rank == 0:
        q_out.put("ok")
    ps.destroy()


def test_dcp_mla_dense_and_sparse_match_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 90
    procs = [ctx.Process(target=_mla_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=180) == "ok"
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
