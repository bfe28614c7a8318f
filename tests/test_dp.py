"""Data-parallel replicas behind one front: same results as one engine, balanced assignment, caller-chosen rank,
a dead replica surfaces as EngineDeadError while the others keep working."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402

KW = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)


def test_data_parallel_front():
    from vllm_metax_b200 import LLM, EngineDeadError, SamplingParams
    from vllm_metax_b200.engine.dp import DataParallelLLM

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (60, 8, 30, 30, 9, 50)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM(tiny_cfg(), **KW).generate(prompts, sp)]
    dp = DataParallelLLM(tiny_cfg(), data_parallel_size=2, **KW)
    try:
        outs = dp.generate(prompts, sp)
        assert [o.outputs[0].token_ids for o in outs] == want
        a = dp.last_assignment
        work = [sum(len(p) + 6 for p, r in zip(prompts, a) if r == k) for k in (0, 1)]
        assert set(a) == {0, 1} and abs(work[0] - work[1]) <= 30, (a, work)
        outs = dp.generate(prompts[:3], sp, dp_rank=1)                      # external load balancing
        assert dp.last_assignment == [1, 1, 1] and [o.outputs[0].token_ids for o in outs] == want[:3]
        with pytest.raises(ValueError):
            dp.generate(prompts[:1], sp, dp_rank=5)
        m = dp.call_all("get_metrics")
        assert len(m) == 2 and m[1]["steps"] > m[0]["steps"] > 0
        # replica 0 dies: calls that need it fail, replica 1 keeps serving
        dp._procs[0].terminate()
        dp._procs[0].join(10)
        with pytest.raises(EngineDeadError):
            dp.generate(prompts, sp)
        assert [o.outputs[0].token_ids for o in dp.generate(prompts[:2], sp, dp_rank=1)] == want[:2]
    finally:
        dp.shutdown()


def test_elastic_scaling_and_healing():
    """Replicas are added and retired between calls, and a replica that died is restarted in place; results never
    change."""
    from vllm_metax_b200 import LLM, EngineDeadError, SamplingParams
    from vllm_metax_b200.engine.dp import DataParallelLLM

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 8, 30, 31, 9, 50)]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in LLM(tiny_cfg(), **KW).generate(prompts, sp)]
    dp = DataParallelLLM(tiny_cfg(), data_parallel_size=1, **KW)
    try:
        assert [o.outputs[0].token_ids for o in dp.generate(prompts, sp)] == want
        assert dp.scale(3) == 3 and len(dp._procs) == 3
        assert [o.outputs[0].token_ids for o in dp.generate(prompts, sp)] == want
        assert set(dp.last_assignment) == {0, 1, 2}
        retired = dp._procs[2]
        assert dp.scale(2) == 2 and not retired.is_alive()
        assert [o.outputs[0].token_ids for o in dp.generate(prompts, sp)] == want
        assert set(dp.last_assignment) == {0, 1}
        with pytest.raises(ValueError):
            dp.scale(0)
        assert dp.scale_events == [(1, 3), (3, 2)]
        # a replica dies and is restarted with the same rank
        dp._procs[1].terminate()
        dp._procs[1].join(10)
        with pytest.raises(EngineDeadError):
            dp.generate(prompts, sp)
        assert dp.heal() == [1]
        assert [o.outputs[0].token_ids for o in dp.generate(prompts, sp)] == want
        assert dp.heal() == []
    finally:
        dp.shutdown()
