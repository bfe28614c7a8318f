"""Sparse decoders that pair the Llama attention block with DeepSeek-style expert blocks.

* ``Glm4MoeForCausalLM`` (GLM-4.5 / 4.6): half-rotary attention with optional per-head q/k norm; sigmoid scores with a
  selection bias, grouped top-k, scaled weights, shared experts, leading dense layers.
* ``DeepseekForCausalLM`` (DeepSeek-MoE 16B): softmax top-k without renormalisation + shared experts.
* ``Ernie4_5_MoeForCausalLM``: softmax scores, bias-corrected selection, renormalised weights, shared experts.

Parity: Glm4MoeForCausalLM / DeepseekForCausalLM / Ernie4_5_MoeForCausalLM rows of the reference's supported-models
table (docs/models/supported_models.md:26-31), served there by upstream model code over its fused-MoE stack.
"""
from __future__ import annotations

from ..config import ModelConfig
from .deepseek_v2 import DeepseekV2MoE
from .qwen3_moe import MoeDecoderLayer, MoeModel, Qwen3MoeForCausalLM


class DsMoeDecoderLayer(MoeDecoderLayer):
    moe_block_cls = DeepseekV2MoE


class DsMoeModel(MoeModel):
    layer_cls = DsMoeDecoderLayer


class _DsMoeForCausalLM(Qwen3MoeForCausalLM):
    model_cls = DsMoeModel
    renames = [(r"\.mlp\.gate\.e_score_correction_bias$", ".mlp.experts.e_score_correction_bias"),
               (r"\.mlp\.moe_statics\.e_score_correction_bias$", ".mlp.experts.e_score_correction_bias")]


class Glm4MoeForCausalLM(_DsMoeForCausalLM):
    def __init__(self, cfg: ModelConfig):
        if "partial_rotary_factor" not in cfg.hf_config and not isinstance(cfg.hf_config.get("rope_parameters"), dict):
            cfg.partial_rotary_factor = 0.5
        super().__init__(cfg)


class DeepseekForCausalLM(_DsMoeForCausalLM):
    pass


class Ernie4_5_MoeForCausalLM(_DsMoeForCausalLM):
    def __init__(self, cfg: ModelConfig):
        cfg.rope_is_neox = False
        cfg.topk_method = "noaux_tc"            # selection by score + bias, weights from the unbiased scores
        cfg.scoring_func = "softmax"
        cfg.norm_topk_prob = True
        cfg.n_group = cfg.topk_group = 1
        super().__init__(cfg)
