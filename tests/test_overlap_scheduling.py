"""Host work of step k + 1 prepared while the device runs step k (``B200_OVERLAP_SCHEDULING``): tokens, stop reasons
and bookkeeping must equal the strictly sequential engine across chunked prefill, stop tokens that end requests
after the next step was already prepared, length limits, pre-emption under a small KV cache and seeded sampling."""
import torch

from vllm_metax_b200 import LLM, SamplingParams
from tests.test_e2e_plumbing import tiny_cfg


def _run(overlap, prompts, sps, **kw):
    args = dict(device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=48, num_gpu_blocks=64)
    args.update(kw)
    llm = LLM(tiny_cfg(), **args)
    llm.engine.overlap_scheduling = overlap
    outs = llm.generate(prompts, sps)
    return llm, [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in outs]


def test_overlapped_steps_match_sequential_engine():
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (5, 70, 33, 120, 1, 48, 17, 90, 60, 9)]
    base = LLM(tiny_cfg(), device="cpu", block_size=16, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=48,
               num_gpu_blocks=64)
    base.engine.overlap_scheduling = False
    probe = base.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    # stop tokens taken from what the model really generates, at different depths, so that requests end by a stop
    # token while the next step (which still holds them) has already been prepared
    sps = []
    for i, o in enumerate(probe):
        toks = o.outputs[0].token_ids
        if i % 3 == 0:
            sps.append(SamplingParams(max_tokens=24, stop_token_ids=[toks[3 + i % 5]]))
        elif i % 3 == 1:
            sps.append(SamplingParams(max_tokens=2 + i, ignore_eos=True))
        else:
            sps.append(SamplingParams(max_tokens=12, ignore_eos=True, temperature=0.9, top_p=0.9, seed=100 + i))
    seq_llm, want = _run(False, prompts, sps)
    ov_llm, got = _run(True, prompts, sps)
    assert got == want
    assert any(reason == "stop" for _, reason in want) and any(reason == "length" for _, reason in want)
    st = ov_llm.engine.stats
    assert st.get("overlapped_steps", 0) > 0 and getattr(ov_llm.engine.runner, "zombie_rows", 0) > 0
    assert seq_llm.engine.stats.get("overlapped_steps", 0) == 0
    assert ov_llm.engine.kv.num_free_blocks == 64 and not ov_llm.engine.scheduler.running       # nothing leaked
    # a second call on the same engine (a stale prepared step must not survive)
    again = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in ov_llm.generate(prompts[:3], sps[:3])]
    assert again == want[:3]


def test_overlapped_steps_with_preemption_and_prefix_cache():
    g = torch.Generator().manual_seed(8)
    shared = torch.randint(0, 1024, (40,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1024, (n,), generator=g).tolist() for n in (10, 30, 3, 22, 15, 8)]
    sps = [SamplingParams(max_tokens=20 + 3 * i, ignore_eos=True) for i in range(len(prompts))]
    kw = dict(num_gpu_blocks=13, enable_prefix_caching=True)       # too few blocks for what is admitted: pre-emptions
    seq_llm, want = _run(False, prompts, sps, **kw)
    ov_llm, got = _run(True, prompts, sps, **kw)
    assert got == want
    assert ov_llm.engine.stats["preemptions"] > 0 and ov_llm.engine.stats.get("overlapped_steps", 0) > 0
    assert ov_llm.engine.kv.num_free_blocks == 13
