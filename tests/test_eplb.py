"""Expert-parallel load balancing: the placement algorithm, the routing maps, the in-place weight shuffle of one
layer, and a tensor-parallel / expert-parallel engine on CPU ranks (gloo) whose experts are re-placed every few
steps while it generates - tokens must equal the run without load balancing."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_metax_b200.parallel import eplb  # noqa: E402


def test_replicate_gives_copies_to_the_hot_experts():
    load = torch.tensor([100, 10, 10, 10, 50, 10, 10, 10])
    cnt = eplb.replicate(load, 12)
    assert int(cnt.sum()) == 12 and int(cnt.min()) == 1
    assert cnt[0] == 4 and cnt[4] == 2            # 100 / 4 = 25 and 50 / 2 = 25: nobody above 25 per copy


@pytest.mark.parametrize("ranks,redundant", [(2, 2), (4, 4), (8, 8)])
def test_rebalance_evens_out_a_skewed_load(ranks, redundant):
    g = torch.Generator().manual_seed(1)
    E = 32
    load = (torch.rand(E, generator=g) ** 4 * 1000).long() + 1       # a few experts take most pairs
    P = E + redundant
    old = eplb.initial_placement(E, P)
    new = eplb.rebalance(load, P, ranks, old)
    assert sorted(set(new.tolist())) == list(range(E))               # every expert is somewhere
    assert new.numel() == P
    before, after = eplb.balancedness(load, old, ranks), eplb.balancedness(load, new, ranks)
    assert after > before and after > 0.8
    # deterministic (every rank computes it on its own) and stable (same statistics -> nothing moves)
    assert torch.equal(new, eplb.rebalance(load, P, ranks, old))
    again = eplb.rebalance(load, P, ranks, new)
    assert torch.equal(again, new)


def test_rebalance_keeps_staying_experts_in_their_slots():
    load = torch.tensor([10, 10, 10, 10, 10, 10, 10, 10])
    old = eplb.initial_placement(8, 8)
    new = eplb.rebalance(load, 8, 2, old)
    moves = eplb.plan_moves(old, new, 2)
    # a flat load needs no more than a few moves; whatever stays on its rank keeps its slot
    per = 4
    for s in range(8):
        e = int(new[s])
        if e in old[(s // per) * per:(s // per + 1) * per].tolist():
            assert int(old[s]) == e
    assert len(moves) <= 4


def test_maps_and_physical_routing():
    from vllm_metax_b200.layers.fused_moe import FusedMoE
    from vllm_metax_b200.parallel import state as ps

    ps.set_eplb(True, 4)
    try:
        m = FusedMoE(8, 2, 32, 16, dtype=torch.float32)
    finally:
        ps.set_eplb(False)
    assert m.eplb and m.num_physical == 12 and m.num_local == 12
    assert m.phy2log.tolist() == list(range(8)) + [0, 1, 2, 3]
    assert m.logcnt.tolist() == [2, 2, 2, 2, 1, 1, 1, 1]
    ids = torch.tensor([[0, 4], [0, 5], [0, 1], [3, 0]], dtype=torch.int32)
    phys = m._to_physical(ids)
    assert torch.equal(m.phy2log[phys.long()].to(torch.int32), ids)          # a slot of the right expert
    assert len(set(phys[:, 0][:3].tolist())) == 2                           # expert 0's pairs alternate between copies
    assert m.expert_load.tolist() == [4, 1, 0, 1, 1, 1, 0, 0]


def _moe_pair(E=8, R=4, H=32, I=16, k=2):
    from vllm_metax_b200.layers.fused_moe import FusedMoE
    from vllm_metax_b200.parallel import state as ps

    torch.manual_seed(0)
    plain = FusedMoE(E, k, H, I, dtype=torch.float32)
    ps.set_eplb(True, R)
    try:
        bal = FusedMoE(E, k, H, I, dtype=torch.float32)
    finally:
        ps.set_eplb(False)
    w1, w3, w2 = torch.randn(E, I, H) * 0.2, torch.randn(E, I, H) * 0.2, torch.randn(E, H, I) * 0.2
    for m in (plain, bal):
        for e in range(E):
            m.weight_loader(m.w13_weight, w1[e], e, "w1")
            m.weight_loader(m.w13_weight, w3[e], e, "w3")
            m.weight_loader(m.w2_weight, w2[e], e, "w2")
    return plain, bal


def test_layer_output_is_unchanged_by_replication_and_by_a_new_placement():
    plain, bal = _moe_pair()
    x = torch.randn(40, 32)
    logits = torch.randn(40, 8)
    logits[:, 5] += 3.0                                                       # expert 5 is hot
    want = plain.forward_reduced(x, logits)
    got = bal.forward_reduced(x, logits)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    assert int(bal.expert_load[5]) >= 30
    new = eplb.rebalance(bal.expert_load.clone(), bal.num_physical, 1, bal.phy2log.long())
    assert int((new == 5).sum()) >= 2                                         # the hot expert is replicated now
    bal.apply_placement(new)
    assert bal.phy2log.tolist() == new.tolist()
    torch.testing.assert_close(bal.forward_reduced(x, logits), want, rtol=1e-5, atol=1e-5)


def _shuffle_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, P = 6, 8
        per = P // world
        old = torch.tensor([0, 1, 2, 3, 4, 5, 0, 1])
        new = torch.tensor([4, 1, 5, 5, 0, 2, 3, 1])          # cross-rank moves, a local move, a slot both read and written
        lo = rank * per
        a = torch.stack([torch.full((3,), float(old[lo + i])) for i in range(per)])
        b = torch.stack([torch.full((2, 2), float(old[lo + i]) * 10) for i in range(per)])
        got = eplb.rearrange_layer([a, b], old, new, list(range(world)), rank)
        ok = all(float(a[i, 0]) == float(new[lo + i]) and float(b[i, 0, 0]) == float(new[lo + i]) * 10 for i in range(per))
        q.put((rank, ok, got))
    finally:
        dist.destroy_process_group()


def test_weight_shuffle_between_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 80)
    procs = [ctx.Process(target=_shuffle_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res), res
    assert sum(n for _, _, n in res) >= 3                      # rows really crossed ranks


tf = pytest.importorskip("transformers")


def _engine_worker(rank, world, port, path, prompts, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=world, block_size=16, max_model_len=128, max_num_seqs=4,
                  max_num_batched_tokens=32, num_gpu_blocks=64, dtype=torch.float32, enable_eplb=True,
                  num_redundant_experts=2, eplb_step_interval=3, eplb_window=3)
        moe = llm.engine.runner.model.model.layers["0"].mlp.experts
        assert moe.eplb and moe.num_physical == 10 and moe.num_local == 10 // world
        outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
        st = llm.engine.stats
        q.put((rank, [o.outputs[0].token_ids for o in outs], st.get("eplb_rearrangements", 0),
               llm.engine.runner.eplb.rows_received, moe.phy2log.tolist()))
    except BaseException as e:
        q.put((rank, repr(e), -1, 0, []))
        raise


def test_engine_with_periodic_replacement_matches_plain_run(tmp_path):
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    cfg = tf.Qwen3MoeConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=256,
                            rms_norm_eps=1e-6, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                            moe_intermediate_size=64, decoder_sparse_step=1, norm_topk_prob=True, mlp_only_layers=[])
    path = str(tmp_path / "ckpt")
    tf.Qwen3MoeForCausalLM(cfg).save_pretrained(path)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 50, 7)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    ref = LLM(path, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              num_gpu_blocks=64, dtype=torch.float32)
    want = [o.outputs[0].token_ids for o in ref.generate(prompts, sp)]
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29990 + (os.getpid() % 150)
    procs = [ctx.Process(target=_engine_worker, args=(r, world, port, path, prompts, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    maps = []
    for rank, toks, rearr, rows, phy2log in got:
        assert rearr >= 0, toks
        assert toks == want, (rank, toks, want)
        assert rearr >= 2                                     # re-placed several times while generating
        maps.append(phy2log)
    assert maps[0] == maps[1]                                 # every rank computed the same placement
    assert sorted(set(maps[0])) == list(range(8))
