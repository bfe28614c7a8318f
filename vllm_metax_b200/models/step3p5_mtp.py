"""Step-3.5 multi-token-prediction module (architecture ``Step3p5MTP``).

Same scheme as the DeepSeek MTP module, over a GQA decoder block and Gemma-style norms (weight + 1):

    x = eh_proj( [ enorm(embed(next_token)) | hnorm(prev_hidden) ] ) -> mtp_block -> shared_head.norm -> head

Checkpoint names: ``model.layers.{L+i}.{enorm,hnorm,eh_proj,shared_head.norm,shared_head.head}`` and the
block under ``model.layers.{L+i}.mtp_block.*``; ``model.embed_tokens`` is shared with the target model.
The block is a dense GQA layer, or a sparse-MoE layer when the config has experts.
Parity: vllm_metax/models/step3p5_mtp.py:28-322 (SharedHead, Step3p5AMultiTokenPredictorLayer,
Step3p5AMultiTokenPredictor, Step3p5MTP.load_weights).
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.attention import PagedGQABackend
from ..layers.basic import GemmaRMSNorm, ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import ReplicatedLinear
from .llama import LlamaDecoderLayer, LlamaForCausalLM
from .qwen3_moe import _EXPERT_RE, _SHARD, MoeDecoderLayer


class SharedHead(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.norm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)


class Step3p5MTPLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, kv_index: int, prefix: str):
        super().__init__()
        self.enorm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.hnorm = GemmaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.eh_proj = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, False, cfg.dtype, prefix=f"{prefix}.eh_proj")
        self.shared_head = SharedHead(cfg)
        block = MoeDecoderLayer if cfg.num_experts else LlamaDecoderLayer
        self.mtp_block = block(cfg, kv_index, f"{prefix}.mtp_block")

    def forward(self, embeds, positions, prev_hidden):
        e = self.enorm(embeds) * (positions > 0).to(embeds.dtype)[:, None]
        x = self.eh_proj(torch.cat([e, self.hnorm(prev_hidden)], dim=-1))
        h, residual = self.mtp_block(positions, x, None)
        return h + residual


class _Body(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        L, n = cfg.num_hidden_layers, max(1, cfg.num_nextn_predict_layers)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.layers = nn.ModuleDict({str(L + i): Step3p5MTPLayer(cfg, i, f"model.layers.{L + i}") for i in range(n)})
        self.first, self.count = L, n


class Step3p5MTP(LlamaForCausalLM):
    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        self.cfg = cfg
        self.model = _Body(cfg)
        self.lm_head = None

    def num_kv_layers(self) -> int:
        return self.model.count

    def kv_cache_spec(self) -> dict:
        return {"kind": "gqa"}

    def allocate_kv_cache(self, num_blocks, block_size, kv_cache_dtype, device):
        from .. import parallel
        from ..parallel import state as ps

        kvh = max(1, self.cfg.num_key_value_heads // ps.tp_size())
        return [PagedGQABackend.allocate(num_blocks, block_size, kvh, self.cfg.head_dim, self.cfg.dtype, kv_cache_dtype,
                                         device) for _ in range(self.model.count)]

    def layer(self, spec_step_idx: int = 0) -> Step3p5MTPLayer:
        return self.model.layers[str(self.model.first + spec_step_idx % self.model.count)]

    def forward(self, input_ids, positions, hidden_states, spec_step_idx: int = 0):
        return self.layer(spec_step_idx)(self.model.embed_tokens(input_ids), positions, hidden_states)

    def compute_logits(self, hidden, spec_step_idx: int = 0):
        head = self.layer(spec_step_idx).shared_head
        return head.head.logits(head.norm(hidden))

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        first, last = self.model.first, self.model.first + self.model.count
        loaded: set[str] = set()
        for name, w in weights:
            if "rotary_emb.inv_freq" in name:
                continue
            parts = name.split(".")
            if name.startswith("model.layers.") and parts[2].isdigit() and not (first <= int(parts[2]) < last):
                continue
            name = name.replace(".transformer.", ".mtp_block.")
            m = _EXPERT_RE.match(name)
            if m is not None:
                mod_name, eid, proj, suffix = m.group(1), int(m.group(2)), m.group(3), m.group(4)
                pname = f"{mod_name}.{'w2' if _SHARD[proj] == 'w2' else 'w13'}_{suffix}"
                if mod_name in modules and pname in params:
                    modules[mod_name].weight_loader(params[pname], w, eid, _SHARD[proj])
                    loaded.add(pname)
                continue
            target, shard = name, None
            for fused, part, sid in self.stacked_params:
                if f".{part}." in name:
                    target, shard = name.replace(part, fused), sid
                    break
            if target not in params:
                continue
            mod = modules[target.rsplit(".", 1)[0]]
            loader = getattr(mod, "weight_loader", None)
            if loader is not None:
                loader(params[target], w, shard)
            else:
                params[target].data.copy_(w.reshape(params[target].shape))
            loaded.add(target)
        for m_ in self.modules():
            qm = getattr(m_, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(m_)
        return loaded
