"""Llama-family dense decoder (Llama 2/3, Mistral, Qwen2, Qwen3) on the B200 kernels.

Layer data flow (all in flat ``[T, hidden]`` token-major tensors):

    (h, res) = fused_add_rms_norm(h, res)            one kernel
    qkv      = tcgen05 GEMM
    RoPE(q,k) + KV-cache write                        one kernel (per-head q/k norm before it for Qwen3)
    attn     = decode kernel | tcgen05 prefill kernel
    h        = o_proj GEMM  (+ TP all-reduce)
    (h, res) = fused_add_rms_norm(h, res)
    h        = down( silu(gate) * up )                2 GEMMs + 1 activation kernel (+ TP all-reduce)

Architecture names follow HF ``config.json``; checkpoints load from HF safetensors with
the usual q/k/v and gate/up stacking.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..attention.metadata import get_forward_context, merge_multimodal_embeddings
from ..layers.attention import Attention
from ..layers.basic import ParallelLMHead, RMSNorm, SiluAndMul, VocabParallelEmbedding, get_rope
from ..layers.linear import GateUpSiluLinear, MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..parallel import state as ps
from ..quantization import get_linear_method


class LlamaMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, intermediate_size: int, prefix: str, reduce_results: bool = True):
        super().__init__()
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        self.fused_act = qm("gate_up_proj") is None and not cfg.mlp_bias and cfg.hidden_act == "silu" and not cfg.enable_lora
        if self.fused_act:
            self.gate_up_proj = GateUpSiluLinear(cfg.hidden_size, intermediate_size, cfg.dtype,
                                                 prefix=f"{prefix}.gate_up_proj")
        else:
            self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [intermediate_size] * 2, cfg.mlp_bias,
                                                           cfg.dtype, qm("gate_up_proj"),
                                                           prefix=f"{prefix}.gate_up_proj")
        self.down_proj = RowParallelLinear(intermediate_size, cfg.hidden_size, cfg.mlp_bias, cfg.dtype,
                                           qm("down_proj"), reduce_results=reduce_results, prefix=f"{prefix}.down_proj")
        self.act = SiluAndMul()

    def activation(self, x):
        """Everything up to (not including) down_proj."""
        return self.gate_up_proj(x) if self.fused_act else self.act(self.gate_up_proj(x))

    def forward(self, x):
        return self.down_proj(self.activation(x))


class LlamaAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        tp = ps.tp_size()
        self.head_dim = cfg.head_dim
        self.total_heads, self.total_kv = cfg.num_attention_heads, cfg.num_key_value_heads
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, self.head_dim, self.total_heads, self.total_kv,
                                          cfg.attention_bias, cfg.dtype, qm("qkv_proj"), prefix=f"{prefix}.qkv_proj")
        self.num_heads, self.num_kv_heads = self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads
        self.q_size, self.kv_size = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.o_proj = RowParallelLinear(self.total_heads * self.head_dim, cfg.hidden_size, cfg.attention_out_bias,
                                        cfg.dtype, qm("o_proj"), prefix=f"{prefix}.o_proj")
        self.rope = get_rope(self.head_dim, int(self.head_dim * cfg.partial_rotary_factor), cfg.max_position_embeddings,
                             cfg.rope_theta, cfg.rope_is_neox, cfg.rope_scaling)
        self.qk_norm = cfg.qk_norm
        if cfg.qk_norm:
            self.q_norm = RMSNorm(self.head_dim, cfg.rms_norm_eps, cfg.dtype)
            self.k_norm = RMSNorm(self.head_dim, cfg.rms_norm_eps, cfg.dtype)
        slopes = None
        if cfg.use_alibi:                              # Baichuan-13B style: linear position bias instead of rotary
            from .gpt import alibi_slopes

            r = ps.tp_rank()
            slopes = alibi_slopes(self.total_heads)[r * self.num_heads: (r + 1) * self.num_heads].contiguous()
            slopes = slopes.to(torch.empty(0).device)
            self.rope = None
        self.attn = Attention(self.num_heads, self.head_dim, self.head_dim ** -0.5, self.num_kv_heads, layer_idx,
                              sliding_window=cfg.sliding_window, alibi_slopes=slopes)

    def attention(self, positions, h):
        """Everything up to (not including) o_proj: ``[T, local_heads * head_dim]``."""
        qkv = self.qkv_proj(h)
        q = qkv[:, : self.q_size]
        k = qkv[:, self.q_size: self.q_size + self.kv_size]
        v = qkv[:, self.q_size + self.kv_size:]
        if self.qk_norm:
            ops.head_rms_norm(q, self.q_norm.weight, self.q_norm.eps, self.num_heads, self.head_dim)
            ops.head_rms_norm(k, self.k_norm.weight, self.k_norm.eps, self.num_kv_heads, self.head_dim)
        sections = getattr(self, "mrope_section", None)
        if sections is not None and self.rope is not None:
            # multimodal rotary positions (Qwen2-VL family): three position streams, see models/qwen2_vl.py
            from ..attention.metadata import get_forward_context
            from .qwen2_vl import apply_mrope

            pos3 = get_forward_context().attn_metadata.extra.get("mrope_positions")
            if pos3 is None:
                pos3 = positions[None, :].expand(3, -1)
            q, k = apply_mrope(q, k, pos3, self.rope.cos_sin_cache, sections, self.head_dim,
                               getattr(self, "mrope_interleaved", False), self.rope.is_neox)
            return self.attn(q, k, v.contiguous(), positions, None)
        return self.attn(q, k, v, positions, self.rope)

    def forward(self, positions, h):
        return self.o_proj(self.attention(positions, h))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        self.self_attn = LlamaAttention(cfg, layer_idx, f"{prefix}.self_attn")
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


class LlamaModel(nn.Module):
    layer_cls = LlamaDecoderLayer

    def __init__(self, cfg: ModelConfig, prefix: str = "model"):
        super().__init__()
        self.cfg = cfg
        if cfg.attention_out_bias or cfg.mlp_bias:     # the fused GEMM + reduce + norm kernel has no bias operand
            self.supports_fused_tp = False
        pp = ps.get_pp_group()
        n = cfg.num_hidden_layers
        per = (n + pp.world_size - 1) // pp.world_size
        self.start_layer = pp.rank_in_group * per
        self.end_layer = min(n, self.start_layer + per)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype) if pp.is_first_rank else None
        self.layers = nn.ModuleDict({str(i): self.layer_cls(cfg, i - self.start_layer, f"{prefix}.layers.{i}")
                                     for i in range(self.start_layer, self.end_layer)})
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype) if pp.is_last_rank else None

    def forward_fused_tp(self, input_ids, positions):
        """Tensor-parallel forward with every row-parallel linear fused with its all-reduce, the residual
        add and the following RMSNorm (``parallel/fused_collectives.py``).  The residual stream is
        sharded by token rows; hidden states between kernels are the all-gathered normalised rows."""
        fused = self.fused_ar
        tp, rank = ps.tp_size(), ps.tp_rank()
        h = merge_multimodal_embeddings(self.embed_tokens(input_ids))
        T = h.shape[0]
        rpr = (T + tp - 1) // tp
        res = torch.zeros(rpr, h.shape[1], dtype=h.dtype, device=h.device)
        n_mine = max(0, min(rpr, T - rank * rpr))
        if n_mine:
            res[:n_mine] = h[rank * rpr: rank * rpr + n_mine]
        layers = [self.layers[str(i)] for i in range(self.start_layer, self.end_layer)]
        x = layers[0].input_layernorm(h)
        for i, lyr in enumerate(layers):
            a = lyr.self_attn.attention(positions, x)
            x = fused(a, lyr.self_attn.o_proj.weight, res, lyr.post_attention_layernorm.weight,
                      lyr.post_attention_layernorm.eps)
            m = lyr.mlp.activation(x)
            nxt = layers[i + 1].input_layernorm if i + 1 < len(layers) else self.norm
            x = fused(m, lyr.mlp.down_proj.weight, res, nxt.weight, nxt.eps)
        return x

    def forward(self, input_ids, positions, intermediate: Optional[dict] = None):
        # large token counts: GEMM + reduce + norm as one NVLink kernel; small ones (decode steps): the split-K GEMMs
        # of the single-GPU path + the peer-store all-reduce are faster than a 128x256-tile kernel on a few tiles
        deep_rows, md = None, None
        if getattr(self, "takes_deepstack", False):       # Qwen3-VL: extra visual feature levels for the first layers
            md = get_forward_context().attn_metadata
            deep_rows = md.extra.get("mm_rows")
        if getattr(self, "fused_ar", None) is not None and input_ids.shape[0] >= getattr(self, "fused_min_tokens", 0) \
                and deep_rows is None:
            return self.forward_fused_tp(input_ids, positions)
        if self.embed_tokens is not None:
            h, residual = merge_multimodal_embeddings(self.embed_tokens(input_ids)), None
        else:
            h, residual = intermediate["hidden_states"], intermediate["residual"]
        deep = md.extra.get("mm_deepstack") if deep_rows is not None else None     # [N, levels, hidden] (DeepStack)
        for i in range(self.start_layer, self.end_layer):
            h, residual = self.layers[str(i)](positions, h, residual)
            if deep is not None and i < deep.shape[1]:
                h.index_add_(0, deep_rows, deep[:, i].to(h.dtype))       # level i joins the stream after layer i
        if self.norm is None:
            return {"hidden_states": h, "residual": residual}
        h, _ = self.norm(h, residual)
        return h


class LlamaForCausalLM(nn.Module):
    model_cls = LlamaModel
    stacked_params = [("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"), ("qkv_proj", "v_proj", "v"),
                      ("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1)]
    # Checkpoint dialects of the same graph: (regex, replacement) pairs applied to every tensor name, and the row order
    # of a qkv tensor that is already fused on disk ("concat": q | k | v; "grouped": per kv head its q heads, k, v).
    renames: list = []
    fused_qkv_layout = "concat"

    def _fused_qkv_rows(self, w: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if self.fused_qkv_layout != "grouped" or w.shape[0] != (H + 2 * Hkv) * D:
            return w
        g, tail = H // Hkv, w.shape[1:]
        x = w.reshape(Hkv, g + 2, D, *tail)
        return torch.cat([x[:, :g].reshape(H * D, *tail), x[:, g].reshape(Hkv * D, *tail),
                          x[:, g + 1].reshape(Hkv * D, *tail)], 0)

    def transform_weight(self, name: str, w: torch.Tensor) -> torch.Tensor:
        """Hook for dialects that store a tensor differently (called with the renamed name)."""
        return w

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.model = self.model_cls(cfg)
        pp = ps.get_pp_group()
        self.lm_head = None
        if pp.is_last_rank:
            if cfg.tie_word_embeddings and self.model.embed_tokens is not None:
                self.lm_head = self.model.embed_tokens
                self.lm_head.__class__ = ParallelLMHead
            else:
                self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)

    # ---- engine interface ---------------------------------------------------
    def num_kv_layers(self) -> int:
        return self.model.end_layer - self.model.start_layer

    def kv_cache_spec(self) -> dict:
        a = next(iter(self.model.layers.values())).self_attn
        return {"kind": "gqa", "num_kv_heads": a.num_kv_heads, "head_size": a.head_dim}

    def forward(self, input_ids, positions, intermediate=None):
        return self.model(input_ids, positions, intermediate)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head.logits(hidden)

    # ---- weights -------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded: set[str] = set()
        for name, w in weights:
            if "rotary_emb.inv_freq" in name or "rotary_pos_emb.inv_freq" in name:
                continue
            for pat, rep in self.renames:
                name = re.sub(pat, rep, name)
            if name.startswith("lm_head.") and self.cfg.tie_word_embeddings:
                continue
            w = self.transform_weight(name, w)
            if ".qkv_proj." in name:
                w = self._fused_qkv_rows(w)
            target, shard = name, None
            for fused, part, sid in self.stacked_params:
                if f".{part}." in name:
                    target, shard = name.replace(part, fused), sid
                    break
            if target not in params:
                continue  # other pipeline stage, or unused tensor
            p = params[target]
            mod = modules[target.rsplit(".", 1)[0]]
            loader = getattr(mod, "weight_loader", None)
            if loader is not None:
                loader(p, w, shard)
            else:
                p.data.copy_(w.reshape(p.shape))
            loaded.add(target)
        for m in self.modules():
            qm = getattr(m, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(m)
        return loaded


# Same graph, different config flags (bias on qkv for Qwen2, per-head q/k norm for Qwen3).
class Qwen2ForCausalLM(LlamaForCausalLM):
    pass


class Qwen3ForCausalLM(LlamaForCausalLM):
    pass


class MistralForCausalLM(LlamaForCausalLM):
    pass
