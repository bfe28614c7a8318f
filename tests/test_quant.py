"""Quantisation ops: per-token-group / per-token / per-tensor fp8, int8, block-scaled fp8 GEMM."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.ops import reference as ref

gpu = pytest.mark.gpu


def cos_diff(a, b):
    a, b = a.float().flatten().cpu(), b.float().flatten().cpu()
    return 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


def make_fp8_weight(N, K, device="cpu"):
    w = torch.randn(N, K) * 0.05
    wb = w.reshape(N // 128, 128, K // 128, 128)
    s = wb.abs().amax(dim=(1, 3)) / 448.0
    q = (wb / s[:, None, :, None]).reshape(N, K).to(torch.float8_e4m3fn)
    return q.to(device), s.float().to(device), w


def test_fp8_linear_method_cpu():
    from vllm_metax_b200.layers.linear import ReplicatedLinear
    from vllm_metax_b200.quantization.fp8 import Fp8BlockLinearMethod

    lin = ReplicatedLinear(256, 384, dtype=torch.float32, quant_method=Fp8BlockLinearMethod())
    q, s, w = make_fp8_weight(384, 256)
    lin.weight.data.copy_(q)
    lin.weight_scale_inv.data.copy_(s)
    x = torch.randn(9, 256)
    assert cos_diff(lin(x), x @ w.t()) < 3e-3


def test_fp8_checkpoint_model_generates_cpu():
    cfg = ModelConfig(architecture="Qwen3MoeForCausalLM", vocab_size=512, hidden_size=256, intermediate_size=256,
                      num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, qk_norm=True,
                      num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, max_position_embeddings=256,
                      dtype=torch.float32, quantization="fp8",
                      quant_config={"quant_method": "fp8", "weight_block_size": [128, 128]})
    llm = LLM(cfg, device="cpu", block_size=16, max_model_len=64, max_num_seqs=2, max_num_batched_tokens=64,
              num_gpu_blocks=16)
    m = llm.engine.runner.model
    assert m.model.layers["0"].self_attn.qkv_proj.weight.dtype == torch.float8_e4m3fn
    assert m.model.layers["0"].mlp.experts.w13_weight.dtype == torch.float8_e4m3fn
    out = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 4


@gpu
@pytest.mark.parametrize("group,ue8m0,col", [(128, False, False), (128, True, False), (64, False, True)])
def test_per_token_group_quant_gpu(group, ue8m0, col, kernel_status_ok):
    x = torch.randn(33, 1024, device="cuda", dtype=torch.bfloat16)
    q, s = ops.per_token_group_quant_fp8(x, group, ue8m0, col)
    wq, ws = ref.per_token_group_quant_fp8(x, group, ue8m0=ue8m0)
    sc = s.t() if col else s
    torch.testing.assert_close(sc, ws, rtol=1e-3, atol=1e-9)
    deq = q.float().reshape(33, -1, group) * sc[..., None]
    wdeq = wq.float().reshape(33, -1, group) * ws[..., None]
    assert cos_diff(deq, wdeq) < 1e-4
    qi, si = ops.per_token_group_quant_int8(x, 128)
    wqi, wsi = ref.per_token_group_quant_int8(x, 128)
    assert cos_diff(qi.float().reshape(33, -1, 128) * si[..., None], wqi.float().reshape(33, -1, 128) * wsi[..., None]) < 1e-4


@gpu
def test_scaled_quant_variants_gpu(kernel_status_ok):
    x = torch.randn(21, 768, device="cuda", dtype=torch.bfloat16)
    q, s = ops.scaled_fp8_quant(x, use_per_token_if_dynamic=True)
    wq, ws = ref.dynamic_per_token_scaled_fp8_quant(x)
    assert cos_diff(q.float() * s, wq.float() * ws) < 1e-4
    q, s = ops.scaled_fp8_quant(x)
    assert cos_diff(q.float() * s, x) < 2e-3
    sc = torch.tensor([0.03], device="cuda")
    q, _ = ops.scaled_fp8_quant(x, sc)
    assert cos_diff(q.float(), ref.static_scaled_fp8_quant(x, sc).float()) < 1e-4
    q, s, _ = ops.scaled_int8_quant(x)
    wq, ws, _ = ref.scaled_int8_quant(x)
    assert (q.int() - wq.int()).abs().max() <= 1
    q, s, z = ops.scaled_int8_quant(x, symmetric=False)
    deq = (q.float() - z.float()) * s
    assert cos_diff(deq, x) < 1e-3


@gpu
def test_merge_attn_states_gpu(kernel_status_ok):
    T, H, D = 19, 8, 128
    a, b = torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16), torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16)
    la, lb = torch.randn(H, T, device="cuda"), torch.randn(H, T, device="cuda")
    lb[:, 3] = float("-inf")
    out, lse = ops.merge_attn_states(a, la, b, lb, want_lse=True)
    wout, wlse = ref.merge_attn_states(a, la, b, lb)
    torch.testing.assert_close(out.float(), wout.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, wlse, rtol=1e-4, atol=1e-4)


@gpu
@pytest.mark.parametrize("M,N,K", [(5, 256, 256), (300, 1536, 1024), (1024, 4096, 7168), (129, 2112, 7168)])
def test_fp8_blockscale_gemm_gpu(M, N, K, kernel_status_ok):
    Np = (N + 127) // 128 * 128
    q, s, w = make_fp8_weight(Np, K, "cuda")
    q, w = q[:N].contiguous(), w[:N]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    xq, xs = ops.per_token_group_quant_fp8(x, 128)
    got = ops.fp8_block_scaled_mm(xq, xs, q, s, torch.bfloat16)
    want = ref.fp8_block_scaled_mm(xq.cpu(), xs.cpu(), q.cpu(), s.cpu(), torch.float32)
    assert cos_diff(got, want) < 1e-4
    assert cos_diff(got, x.float().cpu() @ w.t()) < 3e-3


@gpu
def test_fp8_moe_method_gpu(kernel_status_ok):
    from vllm_metax_b200.layers.fused_moe import FusedMoE
    from vllm_metax_b200.quantization.fp8 import Fp8MoEMethod

    E, H, I, T, k = 8, 512, 256, 100, 2
    with torch.device("cuda"):
        moe = FusedMoE(E, k, H, I, torch.bfloat16, quant_method=Fp8MoEMethod())
    w13 = torch.randn(E, 2 * I, H) * 0.05
    w2 = torch.randn(E, H, I) * 0.05

    def quant(w):
        Eb, N, K = w.shape
        wb = w.reshape(Eb, N // 128, 128, K // 128, 128)
        s = wb.abs().amax(dim=(2, 4)) / 448.0
        return (wb / s[:, :, None, :, None]).reshape(Eb, N, K).to(torch.float8_e4m3fn), s.float()

    q13, s13 = quant(w13)
    q2, s2 = quant(w2)
    moe.w13_weight.data.copy_(q13); moe.w13_weight_scale_inv.data.copy_(s13)
    moe.w2_weight.data.copy_(q2); moe.w2_weight_scale_inv.data.copy_(s2)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    got = moe(x, logits)
    w, ids = ops.topk_gating(logits.cpu(), k, True)
    want = ref.fused_experts(x.cpu().float(), w13, w2, w, ids)
    assert cos_diff(got, want) < 5e-3


def test_scaled_mm_reference_matches_dequant_cpu():
    torch.manual_seed(0)
    M, N, K = 7, 48, 64
    x = torch.randn(M, K)
    w = torch.randn(N, K) * 0.1
    wq = torch.clamp((w / (w.abs().amax(1, keepdim=True) / 127)).round(), -128, 127).to(torch.int8)
    ws = (w.abs().amax(1) / 127)
    # asymmetric per-token activations
    mx, mn = x.amax(1), x.amin(1)
    s = (mx - mn) / 255
    zp = torch.round(-128 - mn / s).int()
    xq = torch.clamp((x / s[:, None]).round() + zp[:, None], -128, 127).to(torch.int8)
    adj = wq.int().sum(1).int()
    out = ops.scaled_mm(xq, wq, s, ws, torch.float32, azp=zp, azp_adj=adj)
    assert cos_diff(out, x @ w.t()) < 2e-3


@gpu
@pytest.mark.parametrize("M,N,K", [(3, 256, 128), (200, 1536, 1024), (1000, 4096, 4096), (129, 2112, 7168), (2048, 4352, 1024)])
@pytest.mark.parametrize("kind", ["int8", "int8_azp", "fp8"])
def test_scaled_mm_gpu(M, N, K, kind, kernel_status_ok):
    torch.manual_seed(1)
    dev = "cuda"
    bias = (torch.randn(N, device=dev) * 0.1).bfloat16()
    if kind == "fp8":
        aq = (torch.randn(M, K, device=dev)).to(torch.float8_e4m3fn)
        wq = (torch.randn(N, K, device=dev)).to(torch.float8_e4m3fn)
        a_s = torch.rand(M, device=dev) * 0.1 + 0.01
        w_s = torch.rand(N, device=dev) * 0.1 + 0.01
        out = ops.scaled_mm(aq, wq, a_s, w_s, torch.bfloat16, bias=bias)
        want = ref.scaled_mm(aq.cpu(), wq.cpu(), a_s.cpu(), w_s.cpu(), torch.float32, bias=bias.cpu())
        assert cos_diff(out, want) < 1e-4
        return
    aq = torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8)
    wq = torch.randint(-128, 128, (N, K), device=dev, dtype=torch.int8)
    a_s = torch.rand(M, device=dev) * 1e-2 + 1e-3
    w_s = torch.rand(N, device=dev) * 1e-2 + 1e-3
    azp = adj = None
    if kind == "int8_azp":
        azp = torch.randint(-20, 20, (M,), device=dev, dtype=torch.int32)
        adj = wq.int().sum(1).int()
    out = ops.scaled_mm(aq, wq, a_s, w_s, torch.bfloat16, azp=azp, azp_adj=adj, bias=bias)
    want = ref.scaled_mm(aq.cpu(), wq.cpu(), a_s.cpu(), w_s.cpu(), torch.float32, None if azp is None else azp.cpu(),
                         None if adj is None else adj.cpu(), bias.cpu())
    # integer accumulation is exact: only the bf16 rounding of the result differs
    torch.testing.assert_close(out.float().cpu(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    assert cos_diff(out, want) < 1e-5


@gpu
def test_scaled_mm_grouped_gpu(kernel_status_ok):
    torch.manual_seed(2)
    dev = "cuda"
    E, N, K, T, topk = 4, 512, 256, 77, 2
    ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).int()
    sorted_ids, block_expert, total_padded = ops.moe_align_block_size(ids, 128, E)
    rows = sorted_ids.numel()
    aq = torch.randint(-128, 128, (rows, K), device=dev, dtype=torch.int8)
    wq = torch.randint(-128, 128, (E, N, K), device=dev, dtype=torch.int8)
    a_s = torch.rand(rows, device=dev) * 1e-2 + 1e-3
    w_s = torch.rand(E, N, device=dev) * 1e-2 + 1e-3
    out = ops.scaled_mm(aq, wq, a_s, w_s, torch.bfloat16, block_expert=block_expert, total_padded=total_padded)
    want = ops.scaled_mm(aq.cpu(), wq.cpu(), a_s.cpu(), w_s.cpu(), torch.float32, block_expert=block_expert.cpu(),
                         total_padded=total_padded.cpu())
    n = int(total_padded.item())
    valid = torch.repeat_interleave(block_expert[: n // 128].cpu() >= 0, 128)
    assert cos_diff(out[:n].cpu()[valid], want[:n][valid]) < 1e-5
