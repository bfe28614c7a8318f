"""Data-parallel attention with experts shared by all replicas (DP attention + EP) on CPU ranks (gloo): every
replica schedules its own prompts, the MoE layers exchange tokens over the dp x tp ranks, and a replica that runs out
of work keeps joining the exchanges with padding steps.  Tokens must equal the single-process run."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

tf = pytest.importorskip("transformers")


def _worker(rank, world, tp, port, path, prompts_by_replica, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams
        from vllm_metax_b200.parallel import state as ps

        llm = LLM(path, device="cpu", tensor_parallel_size=tp, data_parallel_size=world // tp, block_size=16,
                  max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks=64, dtype=torch.float32)
        moe = llm.engine.runner.model.model.layers["0"].mlp.experts
        assert moe.ep == world and moe.num_local == 8 // world and llm.engine.dp_sync
        replica = ps.get_dp_group().rank_in_group
        prompts = prompts_by_replica[replica]
        outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
        q.put((rank, replica, [o.outputs[0].token_ids for o in outs], llm.engine.stats.get("dp_padding_steps", 0)))
    except BaseException as e:
        q.put((rank, -1, repr(e), 0))
        raise


@pytest.mark.parametrize("world,tp", [(2, 1), (4, 2)])
def test_dp_attention_with_shared_experts_matches_single_process(tmp_path, world, tp):
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    cfg = tf.Qwen3MoeConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=256,
                            rms_norm_eps=1e-6, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                            moe_intermediate_size=64, decoder_sparse_step=1, norm_topk_prob=True, mlp_only_layers=[])
    path = str(tmp_path / "ckpt")
    tf.Qwen3MoeForCausalLM(cfg).save_pretrained(path)
    g = torch.Generator().manual_seed(4)
    by_replica = [[torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 50, 7)],      # 50 > one chunk of 32
                  [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5,)]]             # finishes early
    ref = LLM(path, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              num_gpu_blocks=64, dtype=torch.float32)
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    want = [[o.outputs[0].token_ids for o in ref.generate(p, sp)] for p in by_replica]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 150) + world
    procs = [ctx.Process(target=_worker, args=(r, world, tp, port, path, by_replica, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    padded = 0
    for rank, replica, toks, pad in got:
        assert replica >= 0, toks
        assert toks == want[replica], (rank, replica, toks, want[replica])
        padded += pad if replica == 1 else 0
    assert padded > 0          # the short replica kept stepping with padding tokens


def _sp_worker(rank, world, port, path, prompts, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=world, block_size=16, max_model_len=128, max_num_seqs=4,
                  max_num_batched_tokens=32, num_gpu_blocks=64, dtype=torch.float32, use_sequence_parallel_moe=True,
                  all2all_backend="allgather_reducescatter")
        moe = llm.engine.runner.model.model.layers["0"].mlp.experts
        assert moe.sequence_parallel(torch.zeros(4, 128)) and not moe._nvlink_exchange(torch.zeros(4, 128))
        outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
        q.put((rank, [o.outputs[0].token_ids for o in outs], getattr(moe, "_agrs", None) is not None))
    except BaseException as e:
        q.put((rank, repr(e), False))
        raise


def test_sequence_parallel_moe_inside_one_replica(tmp_path):
    """``use_sequence_parallel_moe`` with the collectives backend: every tensor-parallel rank routes its share of the
    tokens, all-gather / reduce-scatter move the rows; same tokens as one process."""
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
    ref = LLM(path, device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              num_gpu_blocks=64, dtype=torch.float32)
    want = [o.outputs[0].token_ids for o in ref.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + (os.getpid() % 40)
    procs = [ctx.Process(target=_sp_worker, args=(r, 2, port, path, prompts, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, toks, used in got:
        assert toks == want, (rank, toks, want)
        assert used                                            # the exchange path ran, not the local filter
    with pytest.raises(ValueError):
        from vllm_metax_b200.parallel import state as ps
        ps.set_moe_parallel(True, "naive")
