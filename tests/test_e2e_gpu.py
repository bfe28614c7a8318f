"""End-to-end on a B200: the bf16 CUDA path (tcgen05 GEMM + attention kernels, CUDA graphs) is
driven in lock step with the fp32 CPU reference engine on the same weights; logits must agree
at every step (prefill, chunked prefill, decode, graph-replayed decode)."""
import time

import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200 import _custom_ops as ops

pytestmark = pytest.mark.gpu


def small_cfg(dtype, **kw):
    d = dict(architecture="LlamaForCausalLM", vocab_size=2048, hidden_size=1024, intermediate_size=2816,
             num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-5,
             rope_theta=10000.0, max_position_embeddings=1024, dtype=dtype, seed=0)
    d.update(kw)
    return ModelConfig(**d)


def step_logits(llm):
    """Run one engine step by hand and return (scheduler_output, logits of sampling rows, requests)."""
    eng = llm.engine
    so = eng.scheduler.schedule()
    r = eng.runner
    md, T, rows, reqs = r._prepare(so)
    with torch.no_grad():
        h = r._forward(md, T)
        logits = r.model.compute_logits(h[torch.tensor(rows, device=h.device)]) if rows else None
    return so, logits, reqs


def lockstep(cpu_llm, gpu_llm, prompts, steps, tol):
    for p in prompts:
        cpu_llm.engine.add_request(p, SamplingParams(max_tokens=64, ignore_eos=True))
        gpu_llm.engine.add_request(p, SamplingParams(max_tokens=64, ignore_eos=True))
    worst = 0.0
    for _ in range(steps):
        so_c, lg_c, reqs_c = step_logits(cpu_llm)
        so_g, lg_g, reqs_g = step_logits(gpu_llm)
        assert [s.num_new_tokens for s in so_c.scheduled] == [s.num_new_tokens for s in so_g.scheduled]
        sampled_c, sampled_g = {}, {}
        if lg_c is not None:
            a, b = lg_c.float(), lg_g.float().cpu()
            cd = 1.0 - torch.nn.functional.cosine_similarity(a, b, dim=-1).min().item()
            worst = max(worst, cd)
            toks = a.argmax(-1).tolist()
            sampled_c = {r.request_id: t for r, t in zip(reqs_c, toks)}
            sampled_g = {r.request_id: t for r, t in zip(reqs_g, toks)}   # CPU tokens drive both engines
        now = time.perf_counter()
        cpu_llm.engine.scheduler.update(so_c, sampled_c, now)
        gpu_llm.engine.scheduler.update(so_g, sampled_g, now)
    torch.cuda.synchronize()
    ops.check_kernel_status(0)
    assert worst < tol, worst


@pytest.mark.parametrize("block_size,budget", [(16, 4096), (64, 96), (128, 4096)])
def test_gpu_engine_tracks_cpu_reference(block_size, budget):
    kw = dict(block_size=block_size, max_model_len=512, max_num_seqs=8, max_num_batched_tokens=budget,
              num_gpu_blocks=256)
    cpu = LLM(small_cfg(torch.float32), device="cpu", **kw)
    gpu = LLM(small_cfg(torch.bfloat16), device="cuda", enforce_eager=True, **kw)
    sd = {k: v.to(torch.bfloat16) for k, v in cpu.engine.runner.model.state_dict().items()}
    gpu.engine.runner.model.load_state_dict(sd)
    # the fp32 engine sees the same (bf16-rounded) weights
    cpu.engine.runner.model.load_state_dict({k: v.float() for k, v in sd.items()})
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (130, 17, 64, 200)]
    lockstep(cpu, gpu, prompts, steps=12, tol=2e-3)


def test_cuda_graph_decode_matches_eager_logits():
    kw = dict(block_size=64, max_model_len=512, max_num_seqs=8, max_num_batched_tokens=1024, num_gpu_blocks=128)
    eager = LLM(small_cfg(torch.bfloat16), device="cuda", enforce_eager=True, **kw)
    graph = LLM(small_cfg(torch.bfloat16), device="cuda", enforce_eager=False, **kw)
    graph.engine.runner.model.load_state_dict(eager.engine.runner.model.state_dict())
    assert graph.engine.runner.graphs, "decode graphs were not captured"
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (33, 90, 7)]
    sp = SamplingParams(max_tokens=1, ignore_eos=True)
    # same first token from both (prefill is eager in both engines)
    a = eager.generate(prompts, sp)
    b = graph.generate(prompts, sp)
    assert [o.outputs[0].token_ids for o in a] == [o.outputs[0].token_ids for o in b]
    # a graph-replayed decode step reproduces the eager logits
    for llm in (eager, graph):
        for p in prompts:
            llm.engine.add_request(p, SamplingParams(max_tokens=8, ignore_eos=True))
        llm.engine.step()  # prefill
    r = graph.engine.runner
    so = graph.engine.scheduler.schedule()
    B = len(so.scheduled)
    bucket = next(x for x in r.buckets if x >= B)
    r._prepare(so, pad_to=bucket)
    gr, glogits, _ = r.graphs[bucket]
    gr.replay()
    so_e, elogits, _ = step_logits(eager)
    torch.cuda.synchronize()
    cs = torch.nn.functional.cosine_similarity(glogits[:B].float(), elogits.float(), dim=-1)
    assert cs.min() > 0.999


def test_generate_api_on_gpu_with_sampling():
    llm = LLM(small_cfg(torch.bfloat16), device="cuda", block_size=64, max_model_len=512, max_num_seqs=16,
              max_num_batched_tokens=2048, num_gpu_blocks=128)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 2048, (40,), generator=g).tolist() for _ in range(6)]
    sps = [SamplingParams(max_tokens=12, temperature=0.8, top_k=50, top_p=0.95, seed=i, ignore_eos=True)
           for i in range(6)]
    o1 = llm.generate(prompts, sps)
    o2 = llm.generate(prompts, sps)
    assert all(len(o.outputs[0].token_ids) == 12 for o in o1)
    assert [o.outputs[0].token_ids for o in o1] == [o.outputs[0].token_ids for o in o2]  # seeded => reproducible
    ops.check_kernel_status(0)
