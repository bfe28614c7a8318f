"""Two more 2-GPU engine tests: data-parallel replicas that share their experts, and prefill context parallelism.
They sort after the rest of the suite: both paths are checked on CPU ranks (tests/test_dp_ep_cpu.py,
tests/test_pcp_cpu.py), but these GPU forms have not yet run to completion on GPUs - the data-parallel one used to
replay CUDA graphs that skipped a host handshake (those engines now run eagerly).  Skipped with fewer than 2 GPUs."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_multigpu import _launch, _ngpu, _tp_checkpoint, _tp_prompts, _tp_single_gpu_tokens  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


# ---- data-parallel attention with experts shared by the replicas ------------------------------------------------
def _dp_ep_worker(rank, world, a2a, path, want):
    os.environ["B200_MOE_A2A"] = "1" if a2a else "0"
    os.environ["B200_FUSED_TP_COLLECTIVES"] = "0"
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200 import _custom_ops as ops
    from vllm_metax_b200.parallel import state as ps

    llm = LLM(path, device="cuda", dtype="bfloat16", data_parallel_size=world, block_size=64, max_model_len=512,
              max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks=64)
    assert llm.engine.dp_sync
    replica = ps.get_dp_group().rank_in_group
    prompts = _dp_ep_prompts()[replica]
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    torch.cuda.synchronize()
    ops.check_kernel_status(rank)
    got = [list(o.outputs[0].token_ids) for o in outs]
    w = want[replica]
    assert [g_[0] for g_ in got] == [x[0] for x in w], (got, w)
    prefix = [next((i for i, (a, b) in enumerate(zip(g_, x)) if a != b), len(x)) for g_, x in zip(got, w)]
    assert min(prefix) >= 2 and sum(prefix) >= 3 * len(w), (prefix, got, w)
    if replica == 1:
        assert llm.engine.stats.get("dp_padding_steps", 0) > 0
    moe = llm.engine.runner.model.model.layers["0"].mlp.experts
    assert (getattr(moe, "_a2a", None) is not None) == a2a           # NVLink dispatch / combine vs all-gather / reduce-scatter
    llm.engine.runner.graphs.clear()


def _dp_ep_prompts():
    g = torch.Generator().manual_seed(12)
    return [[torch.randint(0, 2048, (n,), generator=g).tolist() for n in (100, 300, 33)],
            [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (20,)]]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("a2a", [False, True])
def test_dp2_attention_shared_experts_2gpu(a2a, tmp_path):
    tf = pytest.importorskip("transformers")
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(0)
    cfg = tf.Qwen3MoeConfig(vocab_size=2048, hidden_size=1024, intermediate_size=2048, num_hidden_layers=2,
                            num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024,
                            rms_norm_eps=1e-6, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                            moe_intermediate_size=512, decoder_sparse_step=1, norm_topk_prob=True, mlp_only_layers=[])
    path = str(tmp_path / "ckpt")
    tf.Qwen3MoeForCausalLM(cfg).save_pretrained(path)
    llm = LLM(path, device="cuda", dtype="bfloat16", block_size=64, max_model_len=512, max_num_seqs=8,
              max_num_batched_tokens=256, num_gpu_blocks=64)
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    want = [[list(o.outputs[0].token_ids) for o in llm.generate(p, sp)] for p in _dp_ep_prompts()]
    llm.engine.runner.graphs.clear()
    del llm
    torch.cuda.empty_cache()
    _launch(_dp_ep_worker, 2, a2a, path, want, timeout=300)


# ---- prefill context parallel: two full copies split every prefill chunk ------------------------------------------
def _pcp_engine_worker(rank, world, path, want):
    os.environ["B200_FUSED_TP_COLLECTIVES"] = "0"
    from vllm_metax_b200 import LLM, SamplingParams
    from vllm_metax_b200 import _custom_ops as ops

    llm = LLM(path, device="cuda", dtype="bfloat16", prefill_context_parallel_size=world, block_size=64,
              max_model_len=512, max_num_seqs=8, max_num_batched_tokens=128, num_gpu_blocks=64)
    assert llm.engine.runner.pcp == world
    outs = llm.generate(_tp_prompts(), SamplingParams(max_tokens=16, ignore_eos=True))
    torch.cuda.synchronize()
    ops.check_kernel_status(rank)
    got = [list(o.outputs[0].token_ids) for o in outs]
    # each copy multiplies other token counts than one GPU (other GEMM shapes, bf16): first tokens agree, the rest mostly
    assert [g_[0] for g_ in got] == [w[0] for w in want], (got, want)
    prefix = [next((i for i, (a, b) in enumerate(zip(g_, w)) if a != b), len(w)) for g_, w in zip(got, want)]
    assert min(prefix) >= 2 and sum(prefix) >= 3 * len(want), (prefix, got, want)
    llm.engine.runner.graphs.clear()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pcp2_engine_close_to_single_gpu(tmp_path):
    path = str(tmp_path / "ckpt")
    _tp_checkpoint(path)
    want = _tp_single_gpu_tokens(path)
    _launch(_pcp_engine_worker, 2, path, want, timeout=240)
