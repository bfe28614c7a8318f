"""EAGLE draft head for Llama-family targets: one decoder layer that reads the target's last hidden state together
with the embedding of the token that followed it, ``h = fc([embed(token_{t+1}) ; hidden_t])``, and predicts token
``t + 2`` through the language-model head.

The module has the interface the draft proposer drives (``forward(input_ids, positions, hidden_states)``,
``compute_logits``, ``allocate_kv_cache``), so it plugs into the same lossless verification path as the MTP heads:
``speculative_config={"method": "eagle", "model": <draft checkpoint dir | config dict>}``.  Without ``model`` the
draft shares the target's dimensions (one layer) and, for checkpoints, would be loaded from the target's directory.
Checkpoint names follow the published EAGLE heads: ``fc.*``, ``layers.0.*``, optional ``embed_tokens.*`` /
``lm_head.*`` (taken from the target when absent).
Parity: the speculative-decoding examples of the reference list EAGLE next to MTP and n-gram drafts.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.attention import PagedGQABackend
from ..layers.basic import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import ReplicatedLinear
from .llama import LlamaDecoderLayer, LlamaForCausalLM


class EagleLlamaForCausalLM(nn.Module):
    stacked_params = LlamaForCausalLM.stacked_params

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.fc = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, True, cfg.dtype, prefix="fc")
        self.layers = nn.ModuleDict({"0": LlamaDecoderLayer(cfg, 0, "layers.0")})
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)

    # ---- engine interface ---------------------------------------------------
    def num_kv_layers(self) -> int:
        return 1

    def kv_cache_spec(self) -> dict:
        a = self.layers["0"].self_attn
        return {"kind": "gqa", "num_kv_heads": a.num_kv_heads, "head_size": a.head_dim}

    def allocate_kv_cache(self, num_blocks, block_size, kv_cache_dtype, device):
        spec = self.kv_cache_spec()
        return [PagedGQABackend.allocate(num_blocks, block_size, spec["num_kv_heads"], spec["head_size"], self.cfg.dtype,
                                         kv_cache_dtype, device)]

    def forward(self, input_ids, positions, hidden_states, spec_step_idx: int = 0):
        e = self.embed_tokens(input_ids)
        h = self.fc(torch.cat([e, hidden_states.to(e.dtype)], dim=-1))
        h, residual = self.layers["0"](positions, h, None)
        return h + residual

    def compute_logits(self, hidden: torch.Tensor, spec_step_idx: int = 0) -> torch.Tensor:
        return self.lm_head.logits(hidden)

    def share_with_target(self, target: nn.Module) -> None:
        """Use the target's embedding and head (EAGLE heads ship without them)."""
        inner = getattr(target, "model", target)
        if getattr(inner, "embed_tokens", None) is not None:
            self.embed_tokens = inner.embed_tokens
        if getattr(target, "lm_head", None) is not None:
            self.lm_head = target.lm_head

    # ---- weights -------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded: set[str] = set()
        for name, w in weights:
            name = name[len("model."):] if name.startswith("model.") else name
            if "rotary_emb.inv_freq" in name:
                continue
            target, shard = name, None
            for fused, part, sid in self.stacked_params:
                if f".{part}." in name:
                    target, shard = name.replace(part, fused), sid
                    break
            if target not in params:
                continue
            mod = modules[target.rsplit(".", 1)[0]]
            if hasattr(mod, "weight_loader"):
                mod.weight_loader(params[target], w, shard)
            else:
                params[target].data.copy_(w)
            loaded.add(target)
        return loaded
