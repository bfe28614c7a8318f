"""Weight-only (GPTQ / AWQ / compressed-tensors) and W8A8 int8 quantisation: format conversion,
linear + MoE methods on CPU, the tcgen05 kernels on GPU against the dequantised fp32 oracle."""
import pytest
import torch

from vllm_metax_b200 import LLM, ModelConfig, SamplingParams
from vllm_metax_b200 import _custom_ops as ops
from vllm_metax_b200.quantization import wna16 as W

gpu = pytest.mark.gpu


def cos_diff(a, b):
    a, b = a.float().flatten().cpu(), b.float().flatten().cpu()
    return 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


@pytest.mark.parametrize("bits", [4, 8])
def test_canonical_pack_roundtrip(bits):
    q = torch.randint(0, 1 << bits, (24, 64), dtype=torch.uint8)
    assert torch.equal(W.unpack_canonical(W.pack_canonical(q, bits), bits), q)


def test_nibble_order_matches_kernel_extraction():
    # (word >> 4j) & 0x000F000F must yield elements (2j, 2j+1) in the low / high halves
    q = torch.arange(8, dtype=torch.uint8).reshape(1, 8)
    b = W.pack_canonical(q, 4).to(torch.int64).reshape(-1)
    word = int(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24))
    for j in range(4):
        pair = (word >> (4 * j)) & 0x000F000F
        assert (pair & 0xF, pair >> 16) == (2 * j, 2 * j + 1)


def _gptq_checkpoint(w, bits, group, sym):
    q, s, z = W.quantize_weight(w, bits, group, sym)            # q [N,K], s/z [K/g, N]
    qweight = W.pack_int32(q.t().contiguous(), bits, 0)         # [K/pack, N]
    zstore = (z.to(torch.int64) - 1) & ((1 << bits) - 1)
    qzeros = W.pack_int32(zstore, bits, 1)                      # [K/g, N/pack]
    return qweight, qzeros, s, (q.float() - z.t().repeat_interleave(group, 1)) * s.t().repeat_interleave(group, 1)


def _awq_checkpoint(w, group):
    q, s, z = W.quantize_weight(w, 4, group, False)
    order = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])

    def pk(v_kn):   # [rows, N] -> int32 [rows, N/8] in AWQ nibble order
        v = v_kn.reshape(v_kn.shape[0], -1, 8)[:, :, order].reshape(v_kn.shape[0], -1)
        return W.pack_int32(v, 4, 1)

    deq = (q.float() - z.t().repeat_interleave(group, 1)) * s.t().repeat_interleave(group, 1)
    return pk(q.t().contiguous()), pk(z.to(torch.uint8)), s, deq


@pytest.mark.parametrize("fmt,bits,sym", [("gptq", 4, False), ("gptq", 4, True), ("gptq", 8, False), ("awq", 4, False)])
def test_linear_method_formats_cpu(fmt, bits, sym):
    from vllm_metax_b200.layers.linear import ReplicatedLinear

    torch.manual_seed(0)
    N, K, g = 96, 256, 64
    w = torch.randn(N, K) * 0.1
    lin = ReplicatedLinear(K, N, dtype=torch.float32, quant_method=W.WNA16LinearMethod(fmt, bits, g, sym))
    if fmt == "gptq":
        qweight, qzeros, s, deq = _gptq_checkpoint(w, bits, g, sym)
    else:
        qweight, qzeros, s, deq = _awq_checkpoint(w, g)
    lin.qweight.data.copy_(qweight)
    lin.qzeros.data.copy_(qzeros)
    lin.scales.data.copy_(s)
    lin.quant_method.process_weights_after_loading(lin)
    lin.quant_method.process_weights_after_loading(lin)   # idempotent
    x = torch.randn(5, K)
    torch.testing.assert_close(lin(x), x @ deq.t(), rtol=1e-4, atol=1e-4)
    assert cos_diff(lin(x), x @ w.t()) < (2e-2 if bits == 4 else 1e-3)


def test_gptq_act_order_cpu():
    from vllm_metax_b200.layers.linear import ReplicatedLinear

    torch.manual_seed(1)
    N, K, g = 64, 128, 32
    w = torch.randn(N, K) * 0.1
    perm = torch.randperm(K)
    g_idx = torch.empty(K, dtype=torch.int32)
    g_idx[perm] = (torch.arange(K) // g).int()             # column perm[i] belongs to group i // g
    # quantise with columns gathered group-contiguously, then scatter rows back to checkpoint order
    q, s, z = W.quantize_weight(w[:, perm], 4, g, False)
    q_ckpt = torch.empty_like(q)
    q_ckpt[:, perm] = q
    lin = ReplicatedLinear(K, N, dtype=torch.float32, quant_method=W.WNA16LinearMethod("gptq", 4, g, False, desc_act=True))
    lin.qweight.data.copy_(W.pack_int32(q_ckpt.t().contiguous(), 4, 0))
    lin.qzeros.data.copy_(W.pack_int32((z.to(torch.int64) - 1) & 15, 4, 1))
    lin.scales.data.copy_(s)
    lin.g_idx.data.copy_(g_idx)
    lin.quant_method.process_weights_after_loading(lin)
    x = torch.randn(3, K)
    assert cos_diff(lin(x), x @ w.t()) < 2e-2


def test_int8_linear_method_cpu():
    from vllm_metax_b200.layers.linear import ReplicatedLinear
    from vllm_metax_b200.quantization.int8 import Int8LinearMethod

    torch.manual_seed(2)
    N, K = 48, 128
    w = torch.randn(N, K) * 0.1
    ws = w.abs().amax(1, keepdim=True) / 127
    for sym in (True, False):
        lin = ReplicatedLinear(K, N, bias=True, dtype=torch.float32, quant_method=Int8LinearMethod(act_sym=sym))
        lin.weight.data.copy_(torch.round(w / ws).to(torch.int8))
        lin.weight_loader(lin.weight_scale, ws.reshape(-1))
        lin.bias.data.normal_()
        lin.quant_method.process_weights_after_loading(lin)
        x = torch.randn(6, K) + (0.0 if sym else 1.5)
        assert cos_diff(lin(x), x @ w.t() + lin.bias) < 1e-3


def _tiny_moe_cfg(**kw):
    return ModelConfig(architecture="Qwen3MoeForCausalLM", vocab_size=512, hidden_size=256, intermediate_size=256,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, qk_norm=True,
                       num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, max_position_embeddings=256,
                       dtype=torch.float32, **kw)


@pytest.mark.parametrize("quant,qc", [
    ("gptq", {"quant_method": "gptq", "bits": 4, "group_size": 64, "sym": True}),
    ("awq", {"quant_method": "awq", "bits": 4, "group_size": 64}),
    ("w8a8_int8", {"quant_method": "w8a8_int8"}),
    ("compressed-tensors", {"quant_method": "compressed-tensors", "format": "pack-quantized",
                            "config_groups": {"g0": {"weights": {"num_bits": 4, "group_size": 64, "symmetric": True,
                                                                   "strategy": "group"}}}}),
])
def test_quantised_model_generates_cpu(quant, qc):
    cfg = _tiny_moe_cfg(quantization=quant, quant_config=qc)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=32, block_size=16, seed=0)
    out = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=4, temperature=0.0))
    assert len(out[0].outputs[0].token_ids) == 4


def test_w4a8_int8_activation_experts_cpu():
    """compressed-tensors W4 (channel-wise) + dynamic int8 activations: the nibbles become int8 weights at load and
    the experts run as W8A8; against the dequantised-weight fp32 MoE (the only difference left is the activation
    rounding)."""
    from vllm_metax_b200.layers.fused_moe import FusedMoE, reference_moe
    from vllm_metax_b200.quantization.int8 import W4A8Int8MoEMethod
    from vllm_metax_b200.quantization.wna16 import CompressedTensorsConfig

    qc = CompressedTensorsConfig({"format": "pack-quantized", "config_groups": {"g0": {
        "weights": {"num_bits": 4, "symmetric": True, "strategy": "channel", "group_size": None},
        "input_activations": {"num_bits": 8, "dynamic": True, "symmetric": True, "strategy": "token"}}}})
    method = qc.get_moe_method("model.layers.0.mlp.experts")
    assert isinstance(method, W4A8Int8MoEMethod)
    grouped = CompressedTensorsConfig({"format": "pack-quantized", "config_groups": {"g0": {
        "weights": {"num_bits": 4, "symmetric": True, "strategy": "group", "group_size": 64},
        "input_activations": {"num_bits": 8, "dynamic": True}}}})
    assert not isinstance(grouped.get_moe_method("x"), W4A8Int8MoEMethod)       # group scales: weight-only kernel

    torch.manual_seed(7)
    E, H, I, k = 4, 64, 32, 2
    moe = FusedMoE(E, k, H, I, dtype=torch.float32, quant_method=method)
    deq = {}
    for e in range(E):
        for shard, (n, kk) in (("w1", (I, H)), ("w3", (I, H)), ("w2", (H, I))):
            w = torch.randn(n, kk) * 0.2
            scale = w.abs().amax(1, keepdim=True) / 7
            q = torch.clamp(torch.round(w / scale), -8, 7)
            deq[(e, shard)] = q * scale
            packed = W.pack_int32((q + 8).to(torch.int32), 4, 1)
            assert moe.load_expert_tensor(e, shard, "weight_shape", torch.tensor([n, kk]))
            moe.load_expert_tensor(e, shard, "weight_packed", packed)
            moe.load_expert_tensor(e, shard, "weight_scale", scale.to(torch.bfloat16).float())
            deq[(e, shard)] = q * scale.to(torch.bfloat16).float()
    assert moe.w13_weight.dtype == torch.int8 and int(moe.w13_weight.min()) >= -8 and int(moe.w13_weight.max()) <= 7
    x = torch.randn(24, H)
    logits = torch.randn(24, E)
    got = moe.forward_reduced(x, logits)
    w13 = torch.stack([torch.stack([deq[(e, "w1")], deq[(e, "w3")]], 1).reshape(2 * I, H) for e in range(E)])   # interleaved
    w2 = torch.stack([deq[(e, "w2")] for e in range(E)])
    wts, ids = moe.route(logits)
    want = reference_moe(x, w13, w2, wts, ids)
    assert cos_diff(got, want) < 2e-3


def test_w4a8_checkpoint_config_generates_cpu():
    qc = {"quant_method": "compressed-tensors", "format": "pack-quantized", "config_groups": {"g0": {
        "weights": {"num_bits": 4, "symmetric": True, "strategy": "channel", "group_size": None},
        "input_activations": {"num_bits": 8, "dynamic": True, "symmetric": True, "strategy": "token"}}},
        "ignore": ["re:.*self_attn.*", "lm_head", "re:.*mlp.gate$"]}
    cfg = _tiny_moe_cfg(quantization="compressed-tensors", quant_config=qc)
    llm = LLM(cfg, device="cpu", load_format="dummy", num_gpu_blocks=32, block_size=16, seed=0)
    from vllm_metax_b200.quantization.int8 import W4A8Int8MoEMethod

    assert isinstance(llm.engine.runner.model.model.layers["0"].mlp.experts.quant_method, W4A8Int8MoEMethod)
    out = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=4, temperature=0.0))
    assert len(out[0].outputs[0].token_ids) == 4


# ----------------------------------------------------------------------------- GPU kernels
@gpu
@pytest.mark.parametrize("M,N,K,g", [(1, 256, 256, 128), (7, 4096, 4096, 128), (48, 1536, 2048, 64), (100, 512, 1024, 32),
                                     (300, 2112, 7168, 128), (1000, 4096, 4096, 128)])
@pytest.mark.parametrize("bits,dtype", [(4, torch.bfloat16), (4, torch.float16), (8, torch.bfloat16)])
def test_wna16_gemm_gpu(M, N, K, g, bits, dtype, kernel_status_ok):
    torch.manual_seed(3)
    w = torch.randn(N, K) * 0.05
    q, s, z = W.quantize_weight(w, bits, g, False)
    qc, sc, zc = W.canonical_from_values(q, s, z, bits, dtype)
    x = (torch.randn(M, K) * 0.5).to(dtype)
    bias = (torch.randn(N) * 0.1).to(dtype)
    out = ops.wna16_gemm(x.cuda(), qc.cuda(), sc.cuda(), zc.cuda(), bits, g, bias=bias.cuda())
    want = x.float() @ W.dequantize_canonical(qc, sc, zc, bits, g).to(dtype).float().t() + bias.float()
    assert cos_diff(out, want) < 5e-5
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))


@gpu
@pytest.mark.parametrize("tokens", [6, 200])
def test_wna16_grouped_silu_gate_gpu(tokens, kernel_status_ok):
    torch.manual_seed(4)
    E, H, I, g, topk = 4, 512, 256, 128, 2
    dtype = torch.bfloat16
    w13 = torch.randn(E, 2 * I, H) * 0.05
    w2 = torch.randn(E, H, I) * 0.05
    q13, s13, z13 = W.quantize_weight(w13, 4, g)
    q2, s2, z2 = W.quantize_weight(w2, 4, g)
    c13 = [t.cuda() for t in W.canonical_from_values(q13, s13, z13, 4, dtype)]
    c2 = [t.cuda() for t in W.canonical_from_values(q2, s2, z2, 4, dtype)]
    x = (torch.randn(tokens, H) * 0.5).to(dtype).cuda()
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(tokens)]).int().cuda()
    wts = torch.rand(tokens, topk).cuda()
    tile = ops.wna16_token_tile(tokens * topk // E)
    sorted_ids, block_expert, total, inv = ops.moe_align_block_size(ids, tile, E, None, want_inverse=True)
    a = ops.moe_gather(x, sorted_ids, total, topk)
    h = ops.wna16_gemm(a, *c13, 4, g, block_expert=block_expert, total_padded=total, token_tile=tile, silu_gate=True)
    y = ops.wna16_gemm(h, *c2, 4, g, block_expert=block_expert, total_padded=total, token_tile=tile)
    got = ops.moe_combine(y, wts, inv, tokens, None)
    # oracle: interleaved (gate, up) rows, dequantised weights
    d13 = W.dequantize_canonical(*[t.cpu() for t in c13], 4, g).to(dtype).float()
    d2 = W.dequantize_canonical(*[t.cpu() for t in c2], 4, g).to(dtype).float()
    xf = x.float().cpu()
    want = torch.zeros(tokens, H)
    for t in range(tokens):
        for k in range(topk):
            e = int(ids[t, k])
            hh = (xf[t] @ d13[e].t()).to(dtype).float()
            act = (torch.nn.functional.silu(hh[0::2]) * hh[1::2]).to(dtype).float()
            want[t] += float(wts[t, k]) * (act @ d2[e].t()).to(dtype).float()
    assert cos_diff(got, want) < 1e-4


@gpu
def test_int8_linear_gpu(kernel_status_ok):
    from vllm_metax_b200.layers.linear import ReplicatedLinear
    from vllm_metax_b200.quantization.int8 import Int8LinearMethod

    torch.manual_seed(5)
    N, K = 1024, 2048
    w = torch.randn(N, K) * 0.05
    ws = w.abs().amax(1, keepdim=True) / 127
    for sym in (True, False):
        lin = ReplicatedLinear(K, N, bias=True, dtype=torch.bfloat16, quant_method=Int8LinearMethod(act_sym=sym))
        lin.weight.data.copy_(torch.round(w / ws).to(torch.int8))
        lin.weight_loader(lin.weight_scale, ws.reshape(-1))
        lin.bias.data.normal_()
        lin.quant_method.process_weights_after_loading(lin)
        lin = lin.cuda()
        lin.azp_adj = None if lin.azp_adj is None else lin.azp_adj.cuda()
        x = (torch.randn(77, K) + (0.0 if sym else 1.0)).bfloat16().cuda()
        want = x.float().cpu() @ w.t() + lin.bias.float().cpu()
        assert cos_diff(lin(x), want) < 2e-3
