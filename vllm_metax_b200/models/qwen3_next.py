"""Qwen3-Next: a hybrid decoder - three gated-delta-rule (linear attention) layers for every softmax-attention layer,
each followed by a sparse MoE block with a gated shared expert.

    linear layer   x -> in_proj_qkvz, in_proj_ba
                     -> short causal convolution over [q | k | v] with a per-request carry   (csrc/causal_conv1d.cu)
                     -> gated delta rule, per-request state [Hv, 128, 128] fp32               (csrc/gdn.cu)
                     -> RMSNorm(o) * silu(z) -> out_proj
    full layer     q_proj yields (query, gate) per head; per-head zero-centred q / k norm; a quarter of every head
                   rotated; paged GQA attention (head size 256); output * sigmoid(gate) -> o_proj

The two per-request states of a linear layer live in slot arrays owned by the layer (``allocate_state``); the model
runner hands every scheduled request a slot and says whether the request already has history
(``md.extra["state_indices"]``, ``md.extra["state_has_init"]``), so prefill chunks, decode steps and re-computation
after preemption all go through the same kernels.  Only the full-attention layers own paged KV.

Tensor parallel: k heads (with their share of v heads) are split over the ranks; the checkpoint's per-k-head grouping
of ``in_proj_qkvz`` / ``in_proj_ba`` rows makes that a contiguous row split.

Parity: Qwen3NextForCausalLM in the reference's supported-models table (docs/models/supported_models.md:45) and its
GDN layer glue (vllm_metax/registry/custom_ops/layers/mamba/qwen_gdn_linear_attn.py:16-88).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _custom_ops as ops
from ..attention.metadata import get_forward_context
from ..config import ModelConfig
from ..layers.attention import Attention
from ..layers.basic import RMSNorm, get_rope
from ..layers.linear import ColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..ops import gdn
from ..parallel import state as ps
from ..quantization import get_linear_method
from .llama import LlamaMLP, LlamaModel
from .qwen3_moe import Qwen3MoeForCausalLM, SparseMoeBlock


def layer_is_full_attention(cfg: ModelConfig, i: int) -> bool:
    types = cfg.hf_config.get("layer_types")
    if types:
        return types[i] == "full_attention"
    interval = int(cfg.hf_config.get("full_attention_interval", 4) or 4)
    return (i + 1) % interval == 0


class _ShardedVector(nn.Module):
    """A small parameter split over the TP ranks in named sections (``sections`` = global sizes along dim 0)."""

    def __init__(self, sections: list[int], tail: tuple, dtype, name: str = "weight"):
        super().__init__()
        tp = ps.tp_size()
        assert all(s % tp == 0 for s in sections)
        self.sections, self.pname = sections, name
        self.register_parameter(name, nn.Parameter(torch.zeros(sum(sections) // tp, *tail, dtype=dtype), requires_grad=False))

    def weight_loader(self, param, loaded, shard_id=None):
        tp, r = ps.tp_size(), ps.tp_rank()
        loaded = loaded.reshape(sum(self.sections), *param.shape[1:])
        src = dst = 0
        for s in self.sections:
            n = s // tp
            param.data[dst: dst + n].copy_(loaded[src + r * n: src + (r + 1) * n])
            src += s
            dst += n


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        hf, tp = cfg.hf_config, ps.tp_size()
        self.nv, self.nk = int(hf["linear_num_value_heads"]), int(hf["linear_num_key_heads"])
        self.dk, self.dv = int(hf["linear_key_head_dim"]), int(hf["linear_value_head_dim"])
        self.K = int(hf.get("linear_conv_kernel_dim", 4))
        assert self.nk % tp == 0 and self.nv % self.nk == 0
        self.rep = self.nv // self.nk
        self.nk_l, self.nv_l = self.nk // tp, self.nv // tp
        self.key_l, self.val_l = self.nk_l * self.dk, self.nv_l * self.dv
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        self.in_proj_qkvz = ColumnParallelLinear(cfg.hidden_size, 2 * self.nk * self.dk + 2 * self.nv * self.dv, False,
                                                 cfg.dtype, qm("in_proj_qkvz"), prefix=f"{prefix}.in_proj_qkvz")
        self.in_proj_ba = ColumnParallelLinear(cfg.hidden_size, 2 * self.nv, False, cfg.dtype, None,
                                               prefix=f"{prefix}.in_proj_ba")
        self.conv1d = _ShardedVector([self.nk * self.dk, self.nk * self.dk, self.nv * self.dv], (self.K,), cfg.dtype)
        self.A_log = nn.Parameter(torch.zeros(self.nv_l, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.ones(self.nv_l, dtype=torch.float32), requires_grad=False)
        self.norm = RMSNorm(self.dv, cfg.rms_norm_eps, cfg.dtype)
        self.out_proj = RowParallelLinear(self.nv * self.dv, cfg.hidden_size, False, cfg.dtype, qm("out_proj"),
                                          prefix=f"{prefix}.out_proj")
        self.dtype = cfg.dtype
        self.conv_state: Optional[torch.Tensor] = None
        self.ssm_state: Optional[torch.Tensor] = None

    def weight_loader(self, param, loaded, shard_id=None):       # A_log / dt_bias: one value per (local) v head
        r = ps.tp_rank()
        param.data.copy_(loaded.reshape(-1)[r * self.nv_l: (r + 1) * self.nv_l].to(param.dtype))

    def allocate_state(self, slots: int, device) -> int:
        self.conv_state = torch.zeros(slots, self.K - 1, 2 * self.key_l + self.val_l, dtype=self.dtype, device=device)
        self.ssm_state = torch.zeros(slots, self.nv_l, self.dk, self.dv, dtype=torch.float32, device=device)
        return self.conv_state.numel() * self.conv_state.element_size() + self.ssm_state.numel() * 4

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        md = get_forward_context().attn_metadata
        T = h.shape[0]
        idx, init, qsl = md.extra["state_indices"], md.extra["state_has_init"], md.query_start_loc
        qkvz = self.in_proj_qkvz(h).reshape(T, self.nk_l, 2 * self.dk + 2 * self.rep * self.dv)
        ba = self.in_proj_ba(h).reshape(T, self.nk_l, 2 * self.rep)
        q, k, v, z = qkvz.split([self.dk, self.dk, self.rep * self.dv, self.rep * self.dv], -1)
        b, a = ba.split([self.rep, self.rep], -1)
        mixed = torch.cat([q.reshape(T, self.key_l), k.reshape(T, self.key_l), v.reshape(T, self.val_l)], -1)
        mixed = gdn.causal_conv1d(mixed, self.conv1d.weight, None, self.conv_state, qsl, idx, init, silu=True)
        q, k, v = mixed.split([self.key_l, self.key_l, self.val_l], -1)
        beta = torch.sigmoid(b.reshape(T, self.nv_l).float())
        g = -torch.exp(self.A_log) * F.softplus(a.reshape(T, self.nv_l).float() + self.dt_bias)
        o = gdn.gated_delta_rule(q.reshape(T, self.nk_l, self.dk).contiguous(), k.reshape(T, self.nk_l, self.dk).contiguous(),
                                 v.reshape(T, self.nv_l, self.dv).contiguous(), g, beta, qsl, self.ssm_state, idx, init)
        o = ops.rms_norm(o.reshape(T * self.nv_l, self.dv), self.norm.weight, self.norm.eps)
        o = (o.float() * F.silu(z.reshape(T * self.nv_l, self.dv).float())).to(h.dtype)
        return self.out_proj(o.reshape(T, self.val_l))


class GatedAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, kv_layer_idx: int, prefix: str):
        super().__init__()
        D = self.head_dim = cfg.head_dim
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        # q rows are (query, gate) per head: 2 * H "heads" of size D keep both halves of a head on one rank
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, D, 2 * cfg.num_attention_heads, cfg.num_key_value_heads,
                                          cfg.attention_bias, cfg.dtype, qm("qkv_proj"), prefix=f"{prefix}.qkv_proj")
        self.num_heads, self.num_kv_heads = self.qkv_proj.num_heads // 2, self.qkv_proj.num_kv_heads
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * D, cfg.hidden_size, cfg.attention_bias, cfg.dtype,
                                        qm("o_proj"), prefix=f"{prefix}.o_proj")
        self.q_norm = RMSNorm(D, cfg.rms_norm_eps, cfg.dtype)
        self.k_norm = RMSNorm(D, cfg.rms_norm_eps, cfg.dtype)
        self.rope = get_rope(D, int(D * cfg.partial_rotary_factor), cfg.max_position_embeddings, cfg.rope_theta, True,
                             cfg.rope_scaling)
        self.attn = Attention(self.num_heads, D, D ** -0.5, self.num_kv_heads, kv_layer_idx)

    def forward(self, positions, h):
        T, D, H, Hkv = h.shape[0], self.head_dim, self.num_heads, self.num_kv_heads
        qkv = self.qkv_proj(h)
        qg = qkv[:, : 2 * H * D].reshape(T, H, 2, D)
        q = qg[:, :, 0].reshape(T, H * D)                 # contiguous copies: the kernels want dense head rows
        gate = qg[:, :, 1].reshape(T, H * D)
        k = qkv[:, 2 * H * D: (2 * H + Hkv) * D]
        v = qkv[:, (2 * H + Hkv) * D:]
        ops.head_rms_norm(q, self.q_norm.weight, self.q_norm.eps, H, D)
        ops.head_rms_norm(k, self.k_norm.weight, self.k_norm.eps, Hkv, D)
        o = self.attn(q, k, v, positions, self.rope)
        o = (o.float() * torch.sigmoid(gate.float())).to(h.dtype)
        return self.o_proj(o)


class Qwen3NextDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        i = int(prefix.rsplit(".", 1)[1])
        self.full = layer_is_full_attention(cfg, i)
        if self.full:
            first = i - layer_idx                                   # this stage's first absolute layer
            kv_idx = sum(layer_is_full_attention(cfg, j) for j in range(first, i))
            self.self_attn = GatedAttention(cfg, kv_idx, f"{prefix}.self_attn")
        else:
            self.linear_attn = GatedDeltaNet(cfg, f"{prefix}.linear_attn")
        self.mlp = SparseMoeBlock(cfg, f"{prefix}.mlp") if cfg.layer_is_moe(i) else LlamaMLP(cfg, cfg.intermediate_size, f"{prefix}.mlp")
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)

    def forward(self, positions, h, residual):
        if residual is None:
            residual = h
            h = self.input_layernorm(h)
        else:
            h, residual = self.input_layernorm(h, residual)
        h = self.self_attn(positions, h) if self.full else self.linear_attn(h)
        h, residual = self.post_attention_layernorm(h, residual)
        return self.mlp(h), residual


class Qwen3NextModel(LlamaModel):
    layer_cls = Qwen3NextDecoderLayer
    supports_fused_tp = False


class Qwen3NextForCausalLM(Qwen3MoeForCausalLM):
    model_cls = Qwen3NextModel
    supports_prefix_caching = False        # a cached prefix has KV blocks but no recurrent state to resume from
    stacked_params = [("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"), ("qkv_proj", "v_proj", "v"),
                      ("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1)]

    def __init__(self, cfg: ModelConfig):
        if "partial_rotary_factor" not in cfg.hf_config and not isinstance(cfg.hf_config.get("rope_parameters"), dict):
            cfg.partial_rotary_factor = 0.25
        super().__init__(cfg)

    # ---- engine interface -------------------------------------------------------
    def _layers(self):
        return [self.model.layers[str(i)] for i in range(self.model.start_layer, self.model.end_layer)]

    def num_kv_layers(self) -> int:
        return sum(1 for l in self._layers() if l.full)

    def kv_cache_spec(self) -> dict:
        a = next(l.self_attn for l in self._layers() if l.full)
        return {"kind": "gqa", "num_kv_heads": a.num_kv_heads, "head_size": a.head_dim}

    def allocate_state(self, slots: int, device) -> int:
        """Per-request convolution carry and delta-rule state of every linear layer; returns the bytes taken."""
        return sum(l.linear_attn.allocate_state(slots, device) for l in self._layers() if not l.full)

    # ---- weights ------------------------------------------------------------------
    def transform_weight(self, name: str, w: torch.Tensor) -> torch.Tensor:
        # zero-centred norms ((1 + w) * x_hat) are stored as their effective scale; the gated output norm of the
        # linear layers is an ordinary one
        if name.endswith("norm.weight") and ".linear_attn.norm." not in name:
            return w.float().add(1.0).to(w.dtype)
        if name.endswith(".conv1d.weight"):
            return w.reshape(w.shape[0], w.shape[-1])
        return w
