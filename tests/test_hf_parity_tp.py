"""Tensor-parallel sharding of the newer model families on CPU ranks (gloo, TP2) against Hugging Face: fused-qkv layouts
cut per head group, ALiBi slopes per rank, the delta-rule layer's per-section convolution / per-head parameters, expert
sharding with a gated shared expert."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

tf = pytest.importorskip("transformers")

from tests.test_hf_parity import CASES, PROMPTS  # noqa: E402


def _worker(rank, world, port, path, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), B200_FUSED_TP_COLLECTIVES="0")
    try:
        from vllm_metax_b200 import LLM, SamplingParams

        llm = LLM(path, device="cpu", tensor_parallel_size=world, dtype="float32", max_model_len=128, num_gpu_blocks=32,
                  block_size=16, max_num_batched_tokens=16)
        outs = llm.generate(PROMPTS, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
        q.put((rank, [list(o.outputs[0].token_ids) for o in outs]))
    except BaseException as e:
        q.put((rank, repr(e)))
        raise


@pytest.mark.parametrize("case", ["falcon_grouped", "bloom", "neox", "glm", "qwen3_next_hybrid", "glm4_moe",
                                  "qwen2_moe_shared_expert"])
def test_tp2_matches_hugging_face(case, tmp_path):
    cfg_cls, model_cls, kw = CASES[case]
    torch.manual_seed(0)
    hf = getattr(tf, model_cls)(getattr(tf, cfg_cls)(**kw)).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path))
    want = []
    for ids in PROMPTS:
        with torch.no_grad():
            want.append(hf.generate(torch.tensor([ids]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                                    pad_token_id=0)[0, len(ids):].tolist())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29250 + (os.getpid() % 100) + sorted(CASES).index(case)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == want and got[1] == want, (got, want)
