"""MXFP4 / NVFP4 weight-only checkpoints: packing and scale semantics, and end-to-end loading of a dense and an MoE
model whose outputs must equal the same model loaded from the de-quantised weights."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from vllm_metax_b200.quantization.fp4 import E2M1, dequant_fp4, quant_fp4_ref  # noqa: E402


def test_e2m1_codes_and_scales():
    # byte 0x2B = low nibble 0xB (-1.5), high nibble 0x2 (1.0); UE8M0 exponent 128 = x2
    packed = torch.tensor([[0x2B] * 16], dtype=torch.uint8)
    w = dequant_fp4(packed, torch.tensor([[128]], dtype=torch.uint8), 32, dtype=torch.float32)
    assert w.shape == (1, 32) and w[0, 0] == -3.0 and w[0, 1] == 2.0
    # NVFP4: e4m3 block scale 0.5 per 16, global scale 4 -> x2
    w = dequant_fp4(packed[:, :8], torch.tensor([[0.5]]).to(torch.float8_e4m3fn), 16, torch.tensor(4.0), torch.float32)
    assert w[0, 0] == -3.0 and w[0, 1] == 2.0
    assert len(E2M1) == 8 and E2M1[-1] == 6.0


@pytest.mark.parametrize("kind", ["mxfp4", "nvfp4"])
def test_reference_quantiser_round_trip(kind):
    torch.manual_seed(0)
    w = torch.randn(64, 128) * 0.05
    packed, scale, gs = quant_fp4_ref(w, kind)
    back = dequant_fp4(packed, scale, 32 if kind == "mxfp4" else 16, gs, torch.float32)
    assert packed.shape == (64, 64) and packed.dtype == torch.uint8
    rel = (back - w).norm() / w.norm()
    assert rel < 0.2                                   # 4-bit: ~10 % relative error on gaussian weights
    again = quant_fp4_ref(back, kind)                 # representable values are fixed points
    torch.testing.assert_close(dequant_fp4(again[0], again[1], 32 if kind == "mxfp4" else 16, again[2], torch.float32), back,
                               atol=1e-6, rtol=1e-3)


def _write(path, tensors, cfg):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)


@pytest.mark.parametrize("kind,arch", [("mxfp4", "LlamaForCausalLM"), ("nvfp4", "LlamaForCausalLM"),
                                       ("mxfp4", "Qwen3MoeForCausalLM"), ("nvfp4", "Qwen3MoeForCausalLM")])
def test_fp4_checkpoint_equals_dequantised_checkpoint(tmp_path, kind, arch):
    from vllm_metax_b200 import LLM, SamplingParams

    torch.manual_seed(1)
    H, I, V, L, D = 128, 256, 512, 2, 32
    cfg = dict(architectures=[arch], vocab_size=V, hidden_size=H, intermediate_size=I, num_hidden_layers=L,
               num_attention_heads=4, num_key_value_heads=2, head_dim=D, rms_norm_eps=1e-5, rope_theta=10000.0,
               max_position_embeddings=256, torch_dtype="float32")
    moe = "Moe" in arch
    if moe:
        cfg.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True)
    full = {"model.embed_tokens.weight": torch.randn(V, H) * 0.1, "model.norm.weight": torch.ones(H),
            "lm_head.weight": torch.randn(V, H) * 0.1}
    lin = {}
    for i in range(L):
        p = f"model.layers.{i}."
        full[p + "input_layernorm.weight"] = torch.ones(H)
        full[p + "post_attention_layernorm.weight"] = torch.ones(H)
        if "Qwen3" in arch:
            full[p + "self_attn.q_norm.weight"] = torch.ones(D)
            full[p + "self_attn.k_norm.weight"] = torch.ones(D)
        for n, (o, k) in {"q_proj": (4 * D, H), "k_proj": (2 * D, H), "v_proj": (2 * D, H), "o_proj": (H, 4 * D)}.items():
            lin[p + f"self_attn.{n}"] = torch.randn(o, k) * 0.15
        if moe:
            full[p + "mlp.gate.weight"] = torch.randn(4, H) * 0.3
            for e in range(4):
                for n, (o, k) in {"gate_proj": (64, H), "up_proj": (64, H), "down_proj": (H, 64)}.items():
                    lin[p + f"mlp.experts.{e}.{n}"] = torch.randn(o, k) * 0.15
        else:
            for n, (o, k) in {"gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}.items():
                lin[p + f"mlp.{n}"] = torch.randn(o, k) * 0.15
    qt, dq = dict(full), dict(full)
    group = 32 if kind == "mxfp4" else 16
    for name, w in lin.items():
        packed, scale, gs = quant_fp4_ref(w, kind)
        qt[name + ".weight"] = packed
        qt[name + ".weight_scale"] = scale
        if gs is not None:
            qt[name + ".weight_scale_2"] = gs.reshape(1)
        dq[name + ".weight"] = dequant_fp4(packed, scale, group, gs, torch.float32)
    qcfg = {"quant_method": "mxfp4"} if kind == "mxfp4" else {"quant_method": "modelopt", "quant_algo": "NVFP4"}
    _write(str(tmp_path / "q"), qt, dict(cfg, quantization_config=qcfg))
    _write(str(tmp_path / "d"), dq, cfg)
    kw = dict(dtype="float32", device="cpu", max_model_len=128, num_gpu_blocks=16, block_size=16)
    prompts = [[5, 9, 33, 100, 7, 8, 200, 31, 2, 17], [3, 4, 5]]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    a = LLM(str(tmp_path / "q"), **kw)
    b = LLM(str(tmp_path / "d"), **kw)
    ha, hb = a.embed(prompts, "mean", normalize=False), b.embed(prompts, "mean", normalize=False)
    torch.testing.assert_close(ha, hb, atol=1e-4, rtol=1e-4)
    assert [o.outputs[0].token_ids for o in a.generate(prompts, sp)] == [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
