"""DeepSeek-V2 / V3 / V3.2 (and GLM-MoE-DSA): MLA attention, DeepSeek MoE, V3.2 sparse-attention indexer.

Layer:  input_layernorm -> MLA (q LoRA, latent KV, decoupled RoPE, optional DSA indexer)
        -> post_attention_layernorm -> dense SwiGLU (first_k_dense_replace layers) | MoE with
        grouped sigmoid top-k routing, routed_scaling_factor and shared experts.

Checkpoint layout follows HF: ``q_a_proj`` and ``kv_a_proj_with_mqa`` are loaded into one fused
``fused_qkv_a_proj``; ``kv_b_proj`` is split into ``W_UK`` / ``W_UV`` after loading; experts
``mlp.experts.N.{gate,up,down}_proj`` go to stacked ``w13`` / ``w2``; fp8 checkpoints carry
``weight_scale_inv`` per 128 x 128 block; the indexer's ``wk`` may be stored fp8 and is
dequantised at load.

Parity: vllm_metax/models/deepseek_v2.py:235-1914 (DeepseekV2MLP, DeepseekV2MoE,
DeepseekV2MLAAttention, Indexer :648-796, load_weights :1496-1733, aliases :1905-1914).
"""
from __future__ import annotations

import re
from typing import Iterable, Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.basic import LayerNorm, ParallelLMHead, RMSNorm, VocabParallelEmbedding, get_rope
from ..layers.fused_moe import FusedMoE
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from ..layers.mla import IndexerBackend, MLAAttention, MLABackend, sparse_attn_indexer
from ..ops import reference as ref
from ..parallel import state as ps
from ..quantization import get_linear_method, get_moe_method
from .llama import LlamaMLP


def yarn_mscale(scale: float, mscale: float) -> float:
    import math

    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class DeepseekV2MoE(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, False, cfg.dtype, prefix=f"{prefix}.gate")
        noaux = cfg.topk_method == "noaux_tc"
        self.experts = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size,
                                cfg.dtype, renormalize=cfg.norm_topk_prob, scoring_func=cfg.scoring_func,
                                use_grouped_topk=(cfg.n_group > 1 and cfg.topk_method != "greedy") or noaux, num_expert_group=cfg.n_group,
                                topk_group=cfg.topk_group, routed_scaling_factor=cfg.routed_scaling_factor,
                                e_score_correction_bias=noaux, reduce_results=False,
                                quant_method=get_moe_method(cfg, f"{prefix}.experts"), prefix=f"{prefix}.experts")
        self.shared_experts = None
        if cfg.n_shared_experts:
            self.shared_experts = LlamaMLP(cfg, cfg.moe_intermediate_size * cfg.n_shared_experts,
                                           f"{prefix}.shared_experts", reduce_results=False)

    def forward(self, x):
        shared = self.shared_experts(x) if self.shared_experts is not None else None
        return self.experts.forward_reduced(x, self.gate(x).float(), shared)


class Indexer(nn.Module):
    """DeepSeek-V3.2 lightning indexer: picks ``index_topk`` cache positions per query token."""

    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.n_heads, self.head_dim, self.topk = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        self.rope_dim = cfg.qk_rope_head_dim
        self.wq_b = ReplicatedLinear(cfg.q_lora_rank, self.n_heads * self.head_dim, False, cfg.dtype,
                                     get_linear_method(cfg, f"{prefix}.wq_b"), prefix=f"{prefix}.wq_b")
        self.wk = ReplicatedLinear(cfg.hidden_size, self.head_dim, False, cfg.dtype, prefix=f"{prefix}.wk")
        self.k_norm = LayerNorm(self.head_dim, 1e-6, cfg.dtype)
        self.weights_proj = ReplicatedLinear(cfg.hidden_size, self.n_heads, False, cfg.dtype,
                                             prefix=f"{prefix}.weights_proj")
        self.softmax_scale = self.head_dim ** -0.5

    def forward(self, hidden, q_lora, positions, rope, idx_cache, block_size):
        T = hidden.shape[0]
        q = self.wq_b(q_lora).view(T, self.n_heads, self.head_dim)
        k = self.k_norm(self.wk(hidden))
        # RoPE on the first rope_dim dims of every index head and of k
        qr = q[..., : self.rope_dim].reshape(T, -1).contiguous()
        kr = k[:, : self.rope_dim].contiguous()
        ops.rotary_embedding(positions, qr, kr, self.rope_dim, rope.cos_sin_cache, rope.is_neox)
        q = torch.cat([qr.view(T, self.n_heads, self.rope_dim), q[..., self.rope_dim:]], dim=-1)
        k = torch.cat([kr, k[:, self.rope_dim:]], dim=-1)
        q_fp8, q_scale = ops.per_token_group_quant_fp8(q.reshape(T * self.n_heads, self.head_dim).contiguous(),
                                                       self.head_dim, ue8m0=True)
        weights = self.weights_proj(hidden).float() * q_scale.view(T, self.n_heads) * self.softmax_scale \
            * self.n_heads ** -0.5
        return sparse_attn_indexer(q_fp8.view(T, self.n_heads, self.head_dim), weights, k.contiguous(), idx_cache,
                                   self.topk, block_size)


class DeepseekV2MLAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        tp = ps.tp_size()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.num_heads = cfg.num_attention_heads // tp
        self.nope, self.rope_dim, self.v_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk_dim = self.nope + self.rope_dim
        self.kv_lora, self.q_lora = cfg.kv_lora_rank, cfg.q_lora_rank
        qm = lambda n: get_linear_method(cfg, f"{prefix}.{n}")
        if self.q_lora:
            self.fused_qkv_a_proj = ReplicatedLinear(cfg.hidden_size, self.q_lora + self.kv_lora + self.rope_dim,
                                                     False, cfg.dtype, qm("fused_qkv_a_proj"),
                                                     prefix=f"{prefix}.fused_qkv_a_proj")
            self.q_a_layernorm = RMSNorm(self.q_lora, cfg.rms_norm_eps, cfg.dtype)
            self.q_b_proj = ColumnParallelLinear(self.q_lora, cfg.num_attention_heads * self.qk_dim, False, cfg.dtype,
                                                 qm("q_b_proj"), prefix=f"{prefix}.q_b_proj")
        else:
            self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_attention_heads * self.qk_dim, False,
                                               cfg.dtype, qm("q_proj"), prefix=f"{prefix}.q_proj")
            self.kv_a_proj_with_mqa = ReplicatedLinear(cfg.hidden_size, self.kv_lora + self.rope_dim, False,
                                                       cfg.dtype, qm("kv_a_proj_with_mqa"),
                                                       prefix=f"{prefix}.kv_a_proj_with_mqa")
        self.kv_a_layernorm = RMSNorm(self.kv_lora, cfg.rms_norm_eps, cfg.dtype)
        self.kv_b_proj = ColumnParallelLinear(self.kv_lora, cfg.num_attention_heads * (self.nope + self.v_dim), False,
                                              cfg.dtype, None, prefix=f"{prefix}.kv_b_proj")
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * self.v_dim, cfg.hidden_size, False, cfg.dtype,
                                        qm("o_proj"), prefix=f"{prefix}.o_proj")
        scaling = cfg.rope_scaling
        if scaling and scaling.get("rope_type", scaling.get("type")) in ("yarn", "deepseek_yarn"):
            scaling = dict(scaling, type="deepseek_yarn")
        self.rope = get_rope(self.rope_dim, self.rope_dim, cfg.max_position_embeddings, cfg.rope_theta, False, scaling)
        scale = self.qk_dim ** -0.5
        if scaling and "factor" in scaling:
            m = yarn_mscale(float(scaling["factor"]), float(scaling.get("mscale_all_dim", 0) or 0))
            scale = scale * m * m
        self.attn = MLAAttention(self.num_heads, scale, self.nope, self.rope_dim, self.v_dim, self.kv_lora, layer_idx,
                                 cfg.dtype)
        self.indexer = Indexer(cfg, f"{prefix}.indexer") if cfg.has_indexer else None

    def process_weights_after_loading(self):
        self.attn.set_kv_b(self.kv_b_proj.weight)

    def forward(self, positions, h):
        T = h.shape[0]
        q_lora = None
        if self.q_lora:
            qkv = self.fused_qkv_a_proj(h)
            q_lora = self.q_a_layernorm(qkv[:, : self.q_lora].contiguous())
            kv_a = qkv[:, self.q_lora:]
            q = self.q_b_proj(q_lora)
        else:
            q = self.q_proj(h)
            kv_a = self.kv_a_proj_with_mqa(h)
        kv_c = self.kv_a_layernorm(kv_a[:, : self.kv_lora].contiguous())
        k_pe = kv_a[:, self.kv_lora:].contiguous()
        q = q.view(T, self.num_heads, self.qk_dim)
        q_pe = q[..., self.nope:].reshape(T, -1).contiguous()
        ops.rotary_embedding(positions, q_pe, k_pe, self.rope_dim, self.rope.cos_sin_cache, False)
        q = torch.cat([q[..., : self.nope], q_pe.view(T, self.num_heads, self.rope_dim)], dim=-1)
        topk_idx = None
        if self.indexer is not None:
            from ..attention.metadata import get_forward_context

            ctx = get_forward_context()
            caches = ctx.kv_caches[self.layer_idx]
            topk_idx = self.indexer(h, q_lora, positions, self.rope, caches["idx"], ctx.attn_metadata.block_size)
        a = self.attn(q, kv_c, k_pe, self.kv_b_proj, topk_idx)
        return self.o_proj(a)


class DeepseekV2DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        abs_idx = int(prefix.rsplit(".", 1)[1])
        self.self_attn = DeepseekV2MLAAttention(cfg, layer_idx, f"{prefix}.self_attn")
        self.mlp = DeepseekV2MoE(cfg, f"{prefix}.mlp") if cfg.layer_is_moe(abs_idx) else \
            LlamaMLP(cfg, cfg.intermediate_size, f"{prefix}.mlp")
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


class DeepseekV2Model(nn.Module):
    supports_fused_tp = False

    def __init__(self, cfg: ModelConfig, prefix: str = "model"):
        super().__init__()
        self.cfg = cfg
        pp = ps.get_pp_group()
        n = cfg.num_hidden_layers
        per = (n + pp.world_size - 1) // pp.world_size
        self.start_layer = pp.rank_in_group * per
        self.end_layer = min(n, self.start_layer + per)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype) if pp.is_first_rank else None
        self.layers = nn.ModuleDict({str(i): DeepseekV2DecoderLayer(cfg, i - self.start_layer, f"{prefix}.layers.{i}")
                                     for i in range(self.start_layer, self.end_layer)})
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype) if pp.is_last_rank else None

    def forward(self, input_ids, positions, intermediate=None):
        if self.embed_tokens is not None:
            h, residual = self.embed_tokens(input_ids), None
        else:
            h, residual = intermediate["hidden_states"], intermediate["residual"]
        for i in range(self.start_layer, self.end_layer):
            h, residual = self.layers[str(i)](positions, h, residual)
        if self.norm is None:
            return {"hidden_states": h, "residual": residual}
        h, _ = self.norm(h, residual)
        return h


_EXPERT_RE = re.compile(r"(.*\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.(.+)$")
_SHARD = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}


class DeepseekV2ForCausalLM(nn.Module):
    stacked_params = [("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1)]

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.model = DeepseekV2Model(cfg)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype) if ps.get_pp_group().is_last_rank else None

    # ---- engine interface
    def num_kv_layers(self) -> int:
        return self.model.end_layer - self.model.start_layer

    def kv_cache_spec(self) -> dict:
        return {"kind": "mla", "indexer": self.cfg.has_indexer}

    def kv_bytes_per_block(self, block_size: int, kv_cache_dtype: str) -> int:
        per_tok = 656 if kv_cache_dtype == "fp8_ds_mla" else 576 * 2
        if self.cfg.has_indexer:
            per_tok += self.cfg.index_head_dim + 4
        return per_tok * block_size * self.num_kv_layers()

    def allocate_kv_cache(self, num_blocks, block_size, kv_cache_dtype, device):
        out = []
        for _ in range(self.num_kv_layers()):
            d = {"mla": MLABackend.allocate(num_blocks, block_size, self.cfg.dtype, kv_cache_dtype, device), "idx": None}
            if self.cfg.has_indexer:
                d["idx"] = IndexerBackend.allocate(num_blocks, block_size, self.cfg.index_head_dim, device)
            out.append(d)
        return out

    def forward(self, input_ids, positions, intermediate=None):
        return self.model(input_ids, positions, intermediate)

    def compute_logits(self, hidden):
        return self.lm_head.logits(hidden)

    def finalize_weights(self) -> None:
        for m in self.modules():
            if isinstance(m, DeepseekV2MLAAttention):
                m.process_weights_after_loading()
            qm = getattr(m, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(m)

    # ---- weights
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded: set[str] = set()
        pending_scale: dict[str, torch.Tensor] = {}
        for name, w in weights:
            if "rotary_emb.inv_freq" in name:
                continue
            m = _EXPERT_RE.match(name)
            if m is not None:
                mod_name, eid, proj, suffix = m.group(1), int(m.group(2)), m.group(3), m.group(4)
                if mod_name in modules:
                    shard = _SHARD[proj]
                    pname = f"{mod_name}.{'w2' if shard == 'w2' else 'w13'}_{suffix}"
                    if pname in params:
                        modules[mod_name].weight_loader(params[pname], w, eid, shard)
                        loaded.add(pname)
                    elif modules[mod_name].load_expert_tensor(eid, shard, suffix, w):
                        loaded.add(name)
                continue
            name = name.replace("mlp.gate.e_score_correction_bias", "mlp.experts.e_score_correction_bias")
            # q_a_proj + kv_a_proj_with_mqa -> fused_qkv_a_proj (rows stacked)
            fused_part = None
            if self.cfg.q_lora_rank and ".q_a_proj." in name:
                name, fused_part = name.replace("q_a_proj", "fused_qkv_a_proj"), "q"
            elif self.cfg.q_lora_rank and ".kv_a_proj_with_mqa." in name:
                name, fused_part = name.replace("kv_a_proj_with_mqa", "fused_qkv_a_proj"), "kv"
            # indexer wk stored quantised: dequantise to the parameter dtype at load
            if ".indexer.wk.weight_scale_inv" in name:
                pending_scale[name.replace(".weight_scale_inv", ".weight")] = w
                continue
            target, shard = name, None
            for fused, part, sid in self.stacked_params:
                if f".{part}." in name:
                    target, shard = name.replace(part, fused), sid
                    break
            if target not in params:
                continue
            p = params[target]
            if ".indexer.wk.weight" in target and w.dtype in (torch.float8_e4m3fn, torch.int8):
                sc = pending_scale.get(target)
                if sc is not None:
                    w = ref.dequant_block_fp8_weight(w, sc).to(p.dtype)
                else:
                    w = w.float().to(p.dtype)
            if fused_part is not None:
                ql = self.cfg.q_lora_rank
                is_scale = p.dtype == torch.float32 and getattr(p, "is_scale", False)
                unit = 128 if is_scale else 1
                if fused_part == "q":
                    p.data[: (ql + unit - 1) // unit].copy_(w)
                else:
                    off = ql // unit
                    p.data[off: off + w.shape[0]].copy_(w)
                loaded.add(target)
                continue
            mod = modules[target.rsplit(".", 1)[0]]
            loader = getattr(mod, "weight_loader", None)
            if loader is not None and not target.endswith("e_score_correction_bias"):
                loader(p, w, shard)
            else:
                p.data.copy_(w.reshape(p.shape))
            loaded.add(target)
        self.finalize_weights()
        return loaded


class DeepseekV3ForCausalLM(DeepseekV2ForCausalLM):
    pass


class DeepseekV32ForCausalLM(DeepseekV2ForCausalLM):
    pass


class GlmMoeDsaForCausalLM(DeepseekV2ForCausalLM):
    pass
