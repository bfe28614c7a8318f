"""Pipeline parallel on CPU ranks (gloo): stage 0 sends [hidden | residual] to stage 1, the last stage samples and
broadcasts the tokens; outputs must equal the single-process run of the same checkpoint.  Overlapped mode keeps one
step per stage in flight (asynchronous transfers, requests of a launched step are not scheduled again until its
tokens are back); lock-step mode runs one step at a time."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tests.test_e2e_plumbing import tiny_cfg  # noqa: E402
from tests.test_tp_cpu import export_hf_checkpoint  # noqa: E402


def _params(tp):
    """One seeded random request among greedy ones; with tensor parallelism the logits differ in the last bits from
    the single-process run, so only greedy requests are comparable there."""
    from vllm_metax_b200 import SamplingParams

    mid = (SamplingParams(max_tokens=8, ignore_eos=True, temperature=0.8, top_p=0.9, seed=11) if tp == 1
           else SamplingParams(max_tokens=8, ignore_eos=True))
    return [SamplingParams(max_tokens=8, ignore_eos=True), mid, SamplingParams(max_tokens=5, ignore_eos=True)]


def _worker(rank, world, port, path, prompts, tp, overlap, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0", B200_PP_OVERLAP="1" if overlap else "0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=tp, pipeline_parallel_size=world // tp, block_size=16,
                  max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64, dtype=torch.float32)
        outs = llm.generate(prompts, _params(tp))
        # overlapped: one step per stage was in flight at some point (disjoint request sets); lock-step: never
        assert llm.engine.stats.get("max_inflight", 0) == (world // tp if overlap else 0), llm.engine.stats
        q.put((rank, [o.outputs[0].token_ids for o in outs]))
    except BaseException as e:
        q.put((rank, repr(e)))
        raise


@pytest.mark.parametrize("world,tp,overlap", [(2, 1, True), (2, 1, False), (4, 2, True)])
def test_pipeline_parallel_matches_single_process(tmp_path, world, tp, overlap):
    from vllm_metax_b200 import LLM, SamplingParams

    kw = dict(device="cpu", block_size=16, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks=64)
    ref_llm = LLM(tiny_cfg(num_hidden_layers=3), **kw)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (21, 70, 7)]   # 70 > one scheduler chunk
    want = [o.outputs[0].token_ids for o in ref_llm.generate(prompts, _params(tp))]
    path = str(tmp_path / "ckpt")
    export_hf_checkpoint(ref_llm.engine.runner.model, path)
    import json
    cfg = json.load(open(os.path.join(path, "config.json")))
    cfg["num_hidden_layers"] = 3
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 80) + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, path, prompts, tp, overlap, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):             # every stage ends the run with the same tokens
        assert got[r] == want, (r, got[r])
