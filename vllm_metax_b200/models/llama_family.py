"""Architectures that are the Llama graph under other names or with small twists.

* same tensors, same names: Aquila, InternLM (bias on q/k/v/o), InternLM3, Ernie-4.5 (GPT-J style rotary pairs), Yi ...
* same graph, other checkpoint dialect (tensor names, fused qkv / gate-up tensors): InternLM2 (``wqkv`` grouped per kv
  head), Baichuan (``W_pack``; the 13B models use ALiBi instead of rotary), Qwen-1 (``c_attn``, ``w1`` / ``w2``),
  ChatGLM2/3 + GLM-4 original exports (``query_key_value`` with multi-query groups, ``dense_h_to_4h`` = gate | up);
* GLM (HF port): half-rotary GPT-J pairs, gate_up fused on disk; GLM-4-0414 adds a norm after attention and after the MLP.

Parity: the Llama-like rows of the reference's supported-models table (docs/models/supported_models.md:21-45), which
the reference serves through upstream model code on its kernels.
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..layers.basic import RMSNorm
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaModel


class AquilaForCausalLM(LlamaForCausalLM):
    pass


class InternLMForCausalLM(LlamaForCausalLM):
    pass


class InternLM3ForCausalLM(LlamaForCausalLM):
    pass


class Ernie4_5ForCausalLM(LlamaForCausalLM):
    def __init__(self, cfg: ModelConfig):
        cfg.rope_is_neox = False
        super().__init__(cfg)


class InternLM2ForCausalLM(LlamaForCausalLM):
    fused_qkv_layout = "grouped"
    renames = [(r"^model\.tok_embeddings\.", "model.embed_tokens."), (r"^output\.", "lm_head."),
               (r"\.attention\.wqkv\.", ".self_attn.qkv_proj."), (r"\.attention\.wo\.", ".self_attn.o_proj."),
               (r"\.feed_forward\.w1\.", ".mlp.gate_proj."), (r"\.feed_forward\.w3\.", ".mlp.up_proj."),
               (r"\.feed_forward\.w2\.", ".mlp.down_proj."), (r"\.attention_norm\.", ".input_layernorm."),
               (r"\.ffn_norm\.", ".post_attention_layernorm.")]


class BaichuanForCausalLM(LlamaForCausalLM):
    """Baichuan / Baichuan2 7B: rotary."""
    renames = [(r"\.self_attn\.W_pack\.", ".self_attn.qkv_proj.")]

    def transform_weight(self, name, w):
        if name == "lm_head.weight" and self.cfg.vocab_size == 125696:      # Baichuan2 normalises the head's rows
            return torch.nn.functional.normalize(w.float()).to(w.dtype)
        return w


class BaiChuanForCausalLM(BaichuanForCausalLM):
    """Baichuan / Baichuan2 13B: ALiBi (the 7B checkpoints that carry this name have hidden size 4096 and rotary)."""

    def __init__(self, cfg: ModelConfig):
        cfg.use_alibi = cfg.hidden_size != 4096
        super().__init__(cfg)


class QWenLMHeadModel(LlamaForCausalLM):
    """Qwen-1: ``c_proj(w1(x) * silu(w2(x)))``, so w2 is the gate; the config's intermediate size counts both halves."""
    renames = [(r"^transformer\.wte\.", "model.embed_tokens."), (r"^transformer\.h\.", "model.layers."),
               (r"^transformer\.ln_f\.", "model.norm."), (r"\.ln_1\.", ".input_layernorm."),
               (r"\.ln_2\.", ".post_attention_layernorm."), (r"\.attn\.c_attn\.", ".self_attn.qkv_proj."),
               (r"\.attn\.c_proj\.", ".self_attn.o_proj."), (r"\.mlp\.w2\.", ".mlp.gate_proj."),
               (r"\.mlp\.w1\.", ".mlp.up_proj."), (r"\.mlp\.c_proj\.", ".mlp.down_proj.")]

    def __init__(self, cfg: ModelConfig):
        if not getattr(cfg, "_qwen1_halved", False):
            cfg.intermediate_size //= 2
            cfg._qwen1_halved = True
        super().__init__(cfg)


class GlmForCausalLM(LlamaForCausalLM):
    def __init__(self, cfg: ModelConfig):
        cfg.rope_is_neox = False
        if "partial_rotary_factor" not in cfg.hf_config and not isinstance(cfg.hf_config.get("rope_parameters"), dict):
            cfg.partial_rotary_factor = 0.5
        super().__init__(cfg)


class ChatGLMModel(GlmForCausalLM):
    """ChatGLM2 / ChatGLM3 / GLM-4 in the original export format."""
    renames = [(r"^transformer\.embedding\.word_embeddings\.", "model.embed_tokens."),
               (r"^transformer\.encoder\.layers\.", "model.layers."),
               (r"^transformer\.encoder\.final_layernorm\.", "model.norm."), (r"^transformer\.output_layer\.", "lm_head."),
               (r"\.self_attention\.query_key_value\.", ".self_attn.qkv_proj."),
               (r"\.self_attention\.dense\.", ".self_attn.o_proj."),
               (r"\.mlp\.dense_h_to_4h\.", ".mlp.gate_up_proj."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.down_proj.")]

    def __init__(self, cfg: ModelConfig):
        hf = cfg.hf_config
        cfg.partial_rotary_factor = 0.5
        cfg.rope_theta = 10000.0 * float(hf.get("rope_ratio", 1.0) or 1.0)
        super().__init__(cfg)


ChatGLMForConditionalGeneration = ChatGLMModel


class Glm4DecoderLayer(LlamaDecoderLayer):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__(cfg, layer_idx, prefix)
        self.post_self_attn_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.post_mlp_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)

    def forward(self, positions, h, residual):
        if residual is None:
            residual = h
            h = self.input_layernorm(h)
        else:
            h, residual = self.input_layernorm(h, residual)
        h = self.post_self_attn_layernorm(self.self_attn(positions, h))
        h, residual = self.post_attention_layernorm(h, residual)
        h = self.post_mlp_layernorm(self.mlp(h))
        return h, residual


class Glm4Model(LlamaModel):
    layer_cls = Glm4DecoderLayer
    supports_fused_tp = False      # the branch outputs pass through a norm before they join the residual stream


class Glm4ForCausalLM(GlmForCausalLM):
    model_cls = Glm4Model
