"""Mixture-of-experts: routing, alignment, grouped GEMM pipeline and the Qwen3-MoE model."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.layers.fused_moe import fused_experts, reference_moe
from vllm_metax_b200.ops import reference as ref


def moe_cfg(**kw):
    d = dict(architecture="Qwen3MoeForCausalLM", vocab_size=512, hidden_size=128, intermediate_size=256,
             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, qk_norm=True,
             num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
             max_position_embeddings=256, dtype=torch.float32, seed=0)
    d.update(kw)
    return ModelConfig(**d)


def test_align_gather_combine_roundtrip_cpu():
    T, E, k, H = 37, 8, 2, 64
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    sorted_ids, block_expert, total, inv = ops.moe_align_block_size(ids, 128, E, want_inverse=True)
    assert int(total) % 128 == 0
    flat = ids.reshape(-1)
    for b in range(int(total) // 128):
        rows = sorted_ids[b * 128:(b + 1) * 128]
        valid = rows[rows < T * k].long()
        assert bool((flat[valid] == block_expert[b]).all())
    assert bool((sorted_ids[inv.long()] == torch.arange(T * k, dtype=torch.int32)).all())
    x = torch.randn(T, H)
    a = ops.moe_gather(x, sorted_ids, total, k)
    w = torch.rand(T, k)
    out = ops.moe_combine(a, w, inv, T)
    torch.testing.assert_close(out, x * w.sum(-1, keepdim=True), rtol=1e-5, atol=1e-5)


def test_expert_map_drops_remote_pairs_cpu():
    T, E, k = 20, 8, 2
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[4:8] = torch.arange(4, dtype=torch.int32)
    _, block_expert, total, inv = ops.moe_align_block_size(ids, 128, 4, emap, want_inverse=True)
    remote = ids.reshape(-1) < 4
    assert bool((inv[remote] == -1).all()) and bool((inv[~remote] >= 0).all())


def test_fused_experts_matches_reference_cpu():
    T, E, k, H, I = 50, 8, 2, 64, 32
    x = torch.randn(T, H)
    w13 = torch.randn(E, 2 * I, H) * 0.1
    w2 = torch.randn(E, H, I) * 0.1
    w, ids = ops.topk_gating(torch.randn(T, E), k, True)
    got = fused_experts(x, w13, w2, w, ids, E)
    torch.testing.assert_close(got, reference_moe(x, w13, w2, w, ids), rtol=1e-4, atol=1e-4)
    # two "EP ranks" each computing their half sum to the same result
    parts = []
    for r in range(2):
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[r * 4:(r + 1) * 4] = torch.arange(4, dtype=torch.int32)
        parts.append(fused_experts(x, w13[r * 4:(r + 1) * 4], w2[r * 4:(r + 1) * 4], w, ids, 4, emap))
    torch.testing.assert_close(parts[0] + parts[1], got, rtol=1e-4, atol=1e-4)


def test_qwen3_moe_generates_cpu():
    llm = LLM(moe_cfg(), device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=64,
              num_gpu_blocks=32)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 33)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 6 for o in outs)
    # chunked prefill must not change the result
    llm2 = LLM(moe_cfg(), device="cpu", block_size=16, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=16,
               num_gpu_blocks=32)
    llm2.engine.runner.model.load_state_dict(llm.engine.runner.model.state_dict())
    outs2 = llm2.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    assert [o.outputs[0].token_ids for o in outs] == [o.outputs[0].token_ids for o in outs2]


# ------------------------------------------------------------------ GPU kernels
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("E,k,scoring", [(128, 8, "softmax"), (256, 8, "sigmoid"), (64, 6, "sqrtsoftplus"), (8, 2, "softmax")])
def test_topk_gating_gpu(E, k, scoring, kernel_status_ok):
    g = torch.randn(77, E, device="cuda", dtype=torch.float32)   # fp32: no exact ties between experts
    bias = torch.randn(E, device="cuda") * 0.1 if scoring != "softmax" else None
    w, ids = ops.topk_gating(g, k, True, scoring, bias, 2.5)
    ww, wids = ops.topk_gating(g.cpu().float(), k, True, scoring, None if bias is None else bias.cpu(), 2.5)
    assert torch.equal(ids.cpu().sort(-1)[0], wids.sort(-1)[0])
    torch.testing.assert_close(w.cpu().sort(-1)[0], ww.sort(-1)[0], rtol=2e-2, atol=1e-3)


@gpu
def test_grouped_topk_gpu(kernel_status_ok):
    g = torch.randn(50, 256, device="cuda", dtype=torch.float32)
    bias = torch.randn(256, device="cuda") * 0.1
    w, ids = ops.grouped_topk(g, 8, True, 8, 4, "sigmoid", bias, 2.5)
    ww, wids = ref.grouped_topk(g.cpu(), 8, True, 8, 4, "sigmoid", bias.cpu(), 2.5)
    assert torch.equal(ids.cpu().sort(-1)[0], wids.sort(-1)[0])
    torch.testing.assert_close(w.cpu().sort(-1)[0], ww.sort(-1)[0], rtol=1e-3, atol=1e-4)


@gpu
@pytest.mark.parametrize("T,E,k,H,I", [(300, 16, 4, 1024, 512), (9, 128, 8, 2048, 768), (2000, 8, 2, 512, 1024)])
def test_fused_experts_gpu(T, E, k, H, I, kernel_status_ok):
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    w, ids = ops.topk_gating(torch.randn(T, E, device="cuda"), k, True)
    got = fused_experts(x, w13, w2, w, ids, E)
    want = reference_moe(x.cpu().float(), w13.cpu().float(), w2.cpu().float(), w.cpu(), ids.cpu())
    a, b = got.float().cpu().flatten(), want.flatten()
    assert 1 - float(torch.dot(a, b) / (a.norm() * b.norm())) < 1e-3


@gpu
def test_qwen3_moe_gpu_tracks_cpu(kernel_status_ok):
    cfg = dict(hidden_size=512, head_dim=128, num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=256,
               num_experts=16, num_experts_per_tok=4, vocab_size=1024)
    kw = dict(block_size=64, max_model_len=256, max_num_seqs=4, max_num_batched_tokens=512, num_gpu_blocks=32)
    cpu = LLM(moe_cfg(**cfg), device="cpu", **kw)
    gpu_llm = LLM(moe_cfg(**cfg, dtype=torch.bfloat16), device="cuda", enforce_eager=True, **kw)
    sd = {k: v.to(torch.bfloat16) for k, v in cpu.engine.runner.model.state_dict().items()}
    gpu_llm.engine.runner.model.load_state_dict(sd)
    cpu.engine.runner.model.load_state_dict({k: v.float() for k, v in sd.items()})
    from tests.test_e2e_gpu import lockstep

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (70, 130)]
    lockstep(cpu, gpu_llm, prompts, steps=4, tol=2e-2)


def test_moe_chunked_over_tokens_equals_one_pass(monkeypatch):
    """B200_FUSED_MOE_CHUNK_SIZE: a long step goes through the experts in pieces with the same result."""
    import torch

    from vllm_metax_b200.layers.fused_moe import FusedMoE

    torch.manual_seed(0)
    moe = FusedMoE(8, 2, 32, 16, dtype=torch.float32)
    moe.w13_weight.data.normal_(0, 0.2)
    moe.w2_weight.data.normal_(0, 0.2)
    x, logits, shared = torch.randn(70, 32), torch.randn(70, 8), torch.randn(70, 32)
    want = moe.forward(x, logits, shared)
    monkeypatch.setenv("B200_FUSED_MOE_CHUNK_SIZE", "16")
    torch.testing.assert_close(moe.forward(x, logits, shared), want, rtol=1e-5, atol=1e-5)
    monkeypatch.setenv("B200_FUSED_MOE_CHUNK_SIZE", "0")
    torch.testing.assert_close(moe.forward(x, logits, None), moe.forward(x, logits, shared) - shared, rtol=1e-5, atol=1e-5)
