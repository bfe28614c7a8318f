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
