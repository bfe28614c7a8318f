"""Qwen3-MoE / Qwen2-MoE / Mixtral style sparse decoders.

Attention is the Llama block (per-head q/k RMSNorm for Qwen3); every MoE layer is
``router GEMM -> fused top-k -> FusedMoE`` with experts sharded over the TP/EP ranks.  The
reference runs these architectures through upstream model code on top of its fused-MoE stack
(docs/models/supported_models.md; tests/e2e/test_offline_inference_parallel.py uses
Qwen3-30B-A3B at TP=2).
"""
from __future__ import annotations

import re
from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.basic import RMSNorm
from ..layers.fused_moe import FusedMoE
from ..layers.linear import ReplicatedLinear
from ..quantization import get_moe_method
from .llama import LlamaAttention, LlamaForCausalLM, LlamaMLP, LlamaModel


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, False, cfg.dtype, prefix=f"{prefix}.gate")
        self.experts = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size,
                                cfg.dtype, renormalize=cfg.norm_topk_prob, scoring_func="softmax",
                                reduce_results=False, quant_method=get_moe_method(cfg, f"{prefix}.experts"),
                                prefix=f"{prefix}.experts")
        self.shared_expert = self.shared_expert_gate = None
        if cfg.n_shared_experts:
            width = cfg.shared_expert_intermediate_size or cfg.moe_intermediate_size * cfg.n_shared_experts
            self.shared_expert = LlamaMLP(cfg, width, f"{prefix}.shared_expert", reduce_results=False)
            if cfg.shared_expert_intermediate_size:      # Qwen2-MoE: sigmoid(x . w) scales the shared expert per token
                self.shared_expert_gate = ReplicatedLinear(cfg.hidden_size, 1, False, cfg.dtype,
                                                           prefix=f"{prefix}.shared_expert_gate")

    def _shared(self, x):
        if self.shared_expert is None:
            return None
        y = self.shared_expert(x)
        if self.shared_expert_gate is not None:
            y = (torch.sigmoid(torch.nn.functional.linear(x, self.shared_expert_gate.weight).float()) * y.float()).to(y.dtype)
        return y

    def forward(self, x):
        return self.experts.forward_reduced(x, self.gate(x), self._shared(x))

    def partial(self, x):
        """Un-reduced output (for the fused reduce + norm path)."""
        return self.experts(x, self.gate(x), self._shared(x))


class MoeDecoderLayer(nn.Module):
    moe_block_cls = SparseMoeBlock

    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        abs_idx = int(prefix.rsplit(".", 1)[1])
        self.self_attn = LlamaAttention(cfg, layer_idx, f"{prefix}.self_attn")
        if cfg.layer_is_moe(abs_idx):
            self.mlp = self.moe_block_cls(cfg, f"{prefix}.mlp")
        else:
            self.mlp = LlamaMLP(cfg, cfg.intermediate_size, f"{prefix}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)

    def forward(self, positions, h, residual):
        if residual is None:
            residual = h
            h = self.input_layernorm(h)
        else:
            h, residual = self.input_layernorm(h, residual)
        h = self.self_attn(positions, h)
        h, residual = self.post_attention_layernorm(h, residual)
        h = self.mlp(h)
        return h, residual


class MoeModel(LlamaModel):
    layer_cls = MoeDecoderLayer
    supports_fused_tp = False   # the fused dense-MLP forward does not apply; MoE layers reduce on their own


_EXPERT_RE = re.compile(r"(.*\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.(.+)$")
_SHARD = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2", "w1": "w1", "w3": "w3", "w2": "w2"}


class Qwen3MoeForCausalLM(LlamaForCausalLM):
    model_cls = MoeModel

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        rest = []
        loaded: set[str] = set()
        for name, w in weights:
            name = name.replace("block_sparse_moe", "mlp")
            m = _EXPERT_RE.match(name)
            if m is None:
                rest.append((name, w))
                continue
            mod_name, eid, proj, suffix = m.group(1), int(m.group(2)), m.group(3), m.group(4)
            if mod_name not in modules:
                continue
            shard = _SHARD[proj]
            pname = f"{mod_name}.{'w2' if shard == 'w2' else 'w13'}_{suffix}"
            if pname not in params:
                if modules[mod_name].load_expert_tensor(eid, shard, suffix, w):
                    loaded.add(name)
                continue
            modules[mod_name].weight_loader(params[pname], w, eid, shard)
            loaded.add(pname)
        loaded |= super().load_weights(rest)
        return loaded


class MixtralForCausalLM(Qwen3MoeForCausalLM):
    pass
