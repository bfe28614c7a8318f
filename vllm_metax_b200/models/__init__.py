"""Model registry: HF architecture name -> (module, class), resolved lazily.

Parity: vllm_metax/models/__init__.py:6-38 registers the DeepSeek V2/V3/V3.2/V4, GLM-MoE-DSA
and MTP architectures with vLLM's ModelRegistry; every other architecture of the
reference's supported-models table runs through upstream model code.  Here the registry
also holds the dense / MoE families the benchmark configurations name.
"""
from __future__ import annotations

import importlib

_MODELS: dict[str, tuple[str, str]] = {
    "LlamaForCausalLM": ("llama", "LlamaForCausalLM"),
    "MistralForCausalLM": ("llama", "MistralForCausalLM"),
    "Qwen2ForCausalLM": ("llama", "Qwen2ForCausalLM"),
    "Qwen3ForCausalLM": ("llama", "Qwen3ForCausalLM"),
    "Qwen3MoeForCausalLM": ("qwen3_moe", "Qwen3MoeForCausalLM"),
    "Qwen2MoeForCausalLM": ("qwen3_moe", "Qwen3MoeForCausalLM"),
    "MixtralForCausalLM": ("qwen3_moe", "MixtralForCausalLM"),
    "DeepseekV2ForCausalLM": ("deepseek_v2", "DeepseekV2ForCausalLM"),
    "DeepseekV3ForCausalLM": ("deepseek_v2", "DeepseekV3ForCausalLM"),
    "DeepseekV32ForCausalLM": ("deepseek_v2", "DeepseekV32ForCausalLM"),
    "GlmMoeDsaForCausalLM": ("deepseek_v2", "GlmMoeDsaForCausalLM"),
    "DeepSeekMTPModel": ("deepseek_mtp", "DeepSeekMTP"),
    "DeepseekV4ForCausalLM": ("deepseek_v4", "DeepseekV4ForCausalLM"),
    "DeepSeekV4MTPModel": ("deepseek_v4", "DeepSeekV4MTP"),
    "Step3p5MTP": ("step3p5_mtp", "Step3p5MTP"),
    "EagleLlamaForCausalLM": ("eagle", "EagleLlamaForCausalLM"),
    # the Llama graph under other names / checkpoint dialects
    "AquilaForCausalLM": ("llama_family", "AquilaForCausalLM"),
    "AquilaModel": ("llama_family", "AquilaForCausalLM"),
    "InternLMForCausalLM": ("llama_family", "InternLMForCausalLM"),
    "InternLM2ForCausalLM": ("llama_family", "InternLM2ForCausalLM"),
    "InternLM3ForCausalLM": ("llama_family", "InternLM3ForCausalLM"),
    "Ernie4_5ForCausalLM": ("llama_family", "Ernie4_5ForCausalLM"),
    "BaichuanForCausalLM": ("llama_family", "BaichuanForCausalLM"),
    "BaiChuanForCausalLM": ("llama_family", "BaiChuanForCausalLM"),
    "QWenLMHeadModel": ("llama_family", "QWenLMHeadModel"),
    "GlmForCausalLM": ("llama_family", "GlmForCausalLM"),
    "Glm4ForCausalLM": ("llama_family", "Glm4ForCausalLM"),
    "ChatGLMModel": ("llama_family", "ChatGLMModel"),
    "ChatGLMForConditionalGeneration": ("llama_family", "ChatGLMModel"),
    "LlavaForConditionalGeneration": ("llava", "LlavaForConditionalGeneration"),
    "LlavaNextForConditionalGeneration": ("llava", "LlavaNextForConditionalGeneration"),
    "LlavaOnevisionForConditionalGeneration": ("llava", "LlavaOnevisionForConditionalGeneration"),
    "Qwen2VLForConditionalGeneration": ("qwen2_vl", "Qwen2VLForConditionalGeneration"),
    "Qwen2_5_VLForConditionalGeneration": ("qwen2_vl", "Qwen2_5_VLForConditionalGeneration"),
    "Glm4vForConditionalGeneration": ("qwen2_vl", "Glm4vForConditionalGeneration"),
    "Glm4vMoeForConditionalGeneration": ("qwen2_vl", "Glm4vMoeForConditionalGeneration"),
    "Qwen3VLForConditionalGeneration": ("qwen2_vl", "Qwen3VLForConditionalGeneration"),
    "Qwen3VLMoeForConditionalGeneration": ("qwen2_vl", "Qwen3VLMoeForConditionalGeneration"),
    "InternVLForConditionalGeneration": ("internvl", "InternVLForConditionalGeneration"),
    "InternVLChatModel": ("internvl", "InternVLChatModel"),
    "InternS1ForConditionalGeneration": ("internvl", "InternVLForConditionalGeneration"),    # the same graph, other decoder
    "MambaForCausalLM": ("mamba", "MambaForCausalLM"),
    "Qwen3NextForCausalLM": ("qwen3_next", "Qwen3NextForCausalLM"),
    "Glm4MoeForCausalLM": ("moe_family", "Glm4MoeForCausalLM"),
    "DeepseekForCausalLM": ("moe_family", "DeepseekForCausalLM"),
    "Ernie4_5_MoeForCausalLM": ("moe_family", "Ernie4_5_MoeForCausalLM"),
    # LayerNorm + plain-MLP decoders (rotary, ALiBi or learned positions)
    "GPTNeoXForCausalLM": ("gpt", "GPTNeoXForCausalLM"),
    "FalconForCausalLM": ("gpt", "FalconForCausalLM"),
    "RWForCausalLM": ("gpt", "FalconForCausalLM"),
    "BloomForCausalLM": ("gpt", "BloomForCausalLM"),
    "MPTForCausalLM": ("gpt", "MPTForCausalLM"),
    "MptForCausalLM": ("gpt", "MPTForCausalLM"),
    "GPTBigCodeForCausalLM": ("gpt", "GPTBigCodeForCausalLM"),
    "GPT2LMHeadModel": ("gpt", "GPT2LMHeadModel"),
}


def register_model(arch: str, module: str, cls: str) -> None:
    _MODELS[arch] = (module, cls)


def supported_architectures() -> list[str]:
    return sorted(_MODELS)


def get_model_class(arch: str):
    if arch not in _MODELS:
        raise ValueError(f"unknown architecture {arch!r}; known: {supported_architectures()}")
    mod, cls = _MODELS[arch]
    m = importlib.import_module(mod if "." in mod else f"{__name__}.{mod}")
    return getattr(m, cls)
