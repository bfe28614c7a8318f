"""DeepSeek-V4 family: hyper-connected residual streams (mHC), sqrt-softplus / hash routing MoE, MTP.

What is V4-specific here:

* the residual is ``hc_mult`` parallel streams ``[T, M, H]``; every sub-layer reads a learned mix of them and
  writes back through a Sinkhorn-normalised mixing matrix (``ops/mhc.py``, kernels in ``csrc/mhc.cu``); the
  ``post`` of one sub-layer and the ``pre`` of the next run as one fused kernel, exactly the call pattern of the
  reference's decoder layer;
* routing: ``sqrtsoftplus`` scores with a correction bias, and for the first ``num_hash_layers`` MoE layers a
  token-id hash table (``tid2eid``) picks the experts while the gate only supplies the weights;
* the output head mixes the streams once more (``hc_head``) before the final norm.

Attention: with ``compress_ratios`` in the config the layers run ``layers/v4_attention.py`` (shared 512-wide K = V
vector, sliding window of raw vectors + ratio-c compressed cache with its compressor state, indexer on the ratio-4
layers, attention sink, grouped low-rank output projection).  The raw vectors of all positions stay in the paged
cache (only the last ``sliding_window`` of them are read), so the window's memory saving is not realised yet.
Without ``compress_ratios`` (configs written for the V3.2-style path) the layers run the latent attention of
``deepseek_v2.py`` with the DSA indexer.

Checkpoint names of the V4 release (``layers.N.attn.wq_a`` ...) are rewritten onto the module tree below.
Parity: vllm_metax/models/deepseek_v4/model.py:70-1367 (DeepseekV4MLP, DeepseekV4MoE :478-724 routing,
DeepseekV4DecoderLayer :740-873, DeepseekV4Model :875, DeepseekV4ForCausalLM :1278, weights mapper :1204-1240),
gate_linear.py:9-70, mtp.py:71-531.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.basic import ParallelLMHead, RMSNorm, VocabParallelEmbedding
from ..layers.fused_moe import FusedMoE
from ..layers.linear import ReplicatedLinear
from ..layers.v4_attention import DeepseekV4Attention
from ..ops import mhc
from ..parallel import state as ps
from ..quantization import get_moe_method
from .deepseek_mtp import DeepSeekMTP
from .deepseek_v2 import DeepseekV2ForCausalLM, DeepseekV2MLAAttention
from .llama import LlamaMLP

HC_POST_ALPHA = 2.0


class DeepseekV4MoE(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_abs_idx: int, prefix: str):
        super().__init__()
        self.cfg = cfg
        self.top_k = cfg.num_experts_per_tok
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, False, torch.float32 if cfg.dtype == torch.float32 else cfg.dtype,
                                     prefix=f"{prefix}.gate")
        self.experts = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size,
                                cfg.dtype, renormalize=cfg.norm_topk_prob, scoring_func=cfg.scoring_func,
                                use_grouped_topk=False, routed_scaling_factor=cfg.routed_scaling_factor,
                                e_score_correction_bias=True, reduce_results=False,
                                quant_method=get_moe_method(cfg, f"{prefix}.experts"), prefix=f"{prefix}.experts")
        self.hash_routed = layer_abs_idx < cfg.num_hash_layers
        if self.hash_routed:
            self.register_buffer("tid2eid", torch.zeros(cfg.vocab_size, self.top_k, dtype=torch.int32), persistent=True)
        self.shared_experts = None
        if cfg.n_shared_experts:
            self.shared_experts = LlamaMLP(cfg, cfg.moe_intermediate_size * cfg.n_shared_experts,
                                           f"{prefix}.shared_experts", reduce_results=False)

    def _hash_route(self, logits: torch.Tensor, input_ids: torch.Tensor):
        """Experts come from the token-id table; weights are the gate's scores of those experts."""
        ids = self.tid2eid[input_ids.long()]
        x = logits.float()
        if self.cfg.scoring_func == "sqrtsoftplus":
            sc = torch.sqrt(torch.nn.functional.softplus(x))
        elif self.cfg.scoring_func == "sigmoid":
            sc = torch.sigmoid(x)
        else:
            sc = torch.softmax(x, -1)
        w = sc.gather(1, ids.long())
        if self.cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        return (w * self.cfg.routed_scaling_factor).float(), ids.int()

    def forward(self, x: torch.Tensor, input_ids: torch.Tensor) -> torch.Tensor:
        shared = self.shared_experts(x) if self.shared_experts is not None else None
        logits = self.gate(x.to(self.gate.weight.dtype)).float()
        e = self.experts
        if self.hash_routed:
            w, ids = self._hash_route(logits, input_ids)
            if e.quant_method is not None:
                y = e.quant_method.apply(e, x, w, ids, shared)
            else:
                from ..layers.fused_moe import fused_experts

                y = fused_experts(x, e.w13_weight, e.w2_weight, w, ids, e.num_local, e.expert_map, shared)
        else:
            return e.forward_reduced(x, logits, shared)
        if ps.tp_size() > 1:
            y = ps.tensor_model_parallel_all_reduce(y)
        return y


class _HcParams(nn.Module):
    """fn / base / scale of one mHC site."""

    def __init__(self, m: int, hidden: int, head: bool = False):
        super().__init__()
        nmix = m if head else (2 + m) * m
        self.fn = nn.Parameter(torch.zeros(nmix, m * hidden, dtype=torch.float32), requires_grad=False)
        self.base = nn.Parameter(torch.zeros(nmix, dtype=torch.float32), requires_grad=False)
        self.scale = nn.Parameter(torch.ones(1 if head else 3, dtype=torch.float32), requires_grad=False)


class DeepseekV4DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, kv_index: int, prefix: str):
        super().__init__()
        abs_idx = int(prefix.rsplit(".", 1)[1])
        self.cfg = cfg
        self.attn = (DeepseekV4Attention(cfg, kv_index, f"{prefix}.attn") if cfg.compress_ratios is not None
                     else DeepseekV2MLAAttention(cfg, kv_index, f"{prefix}.attn"))
        self.ffn = DeepseekV4MoE(cfg, abs_idx, f"{prefix}.ffn") if cfg.layer_is_moe(abs_idx) else \
            LlamaMLP(cfg, cfg.intermediate_size, f"{prefix}.ffn")
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)
        self.hc_attn = _HcParams(cfg.hc_mult, cfg.hidden_size)
        self.hc_ffn = _HcParams(cfg.hc_mult, cfg.hidden_size)

    def _args(self, hc: _HcParams):
        c = self.cfg
        return (hc.fn, hc.scale, hc.base, c.rms_norm_eps, c.hc_eps, c.hc_eps, HC_POST_ALPHA, c.hc_sinkhorn_iters)

    def forward(self, x, positions, input_ids, post, comb, residual):
        if residual is None:
            residual = x                                    # [T, M, H] streams
            post, comb, x = mhc.mhc_pre(residual, *self._args(self.hc_attn))
        else:
            residual, post, comb, x = mhc.mhc_fused_post_pre(x, residual, post, comb, *self._args(self.hc_attn))
        x = self.attn(positions, self.attn_norm(x))
        residual, post, comb, x = mhc.mhc_fused_post_pre(x, residual, post, comb, *self._args(self.hc_ffn))
        x = self.ffn_norm(x)
        x = self.ffn(x, input_ids) if isinstance(self.ffn, DeepseekV4MoE) else self.ffn(x)
        return x, residual, post, comb


class DeepseekV4Model(nn.Module):
    supports_fused_tp = False

    def __init__(self, cfg: ModelConfig, prefix: str = "model"):
        super().__init__()
        assert 1 <= cfg.hc_mult <= 4, "hc_mult must be 1..4"
        self.cfg = cfg
        self.start_layer, self.end_layer = 0, cfg.num_hidden_layers
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.layers = nn.ModuleDict({str(i): DeepseekV4DecoderLayer(cfg, i, f"{prefix}.layers.{i}")
                                     for i in range(cfg.num_hidden_layers)})
        self.hc_head = _HcParams(cfg.hc_mult, cfg.hidden_size, head=True)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype)

    def forward(self, input_ids, positions, intermediate=None):
        x = mhc.expand_to_streams(self.embed_tokens(input_ids), self.cfg.hc_mult)
        post = comb = residual = None
        for i in range(self.cfg.num_hidden_layers):
            x, residual, post, comb = self.layers[str(i)](x, positions, input_ids, post, comb, residual)
        residual = mhc.mhc_post(x, residual, post, comb)
        c = self.cfg
        h = mhc.mhc_head(residual, self.hc_head.fn, self.hc_head.scale, self.hc_head.base, c.rms_norm_eps, c.hc_eps)
        return self.norm(h)


# V4 release names -> module tree of this file
_RENAMES = (
    (".attn.wq_a.", ".attn.q_a_proj."), (".attn.wq_b.", ".attn.q_b_proj."), (".attn.wq.", ".attn.q_proj."),
    (".attn.wkv_a.", ".attn.kv_a_proj_with_mqa."), (".attn.wkv_b.", ".attn.kv_b_proj."), (".attn.wo.", ".attn.o_proj."),
    (".attn.q_norm.", ".attn.q_a_layernorm."), (".attn.kv_norm.", ".attn.kv_a_layernorm."),
    (".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj."),
    (".ffn.gate.bias", ".ffn.experts.e_score_correction_bias"),
    (".hc_attn_fn", ".hc_attn.fn"), (".hc_attn_base", ".hc_attn.base"), (".hc_attn_scale", ".hc_attn.scale"),
    (".hc_ffn_fn", ".hc_ffn.fn"), (".hc_ffn_base", ".hc_ffn.base"), (".hc_ffn_scale", ".hc_ffn.scale"),
    ("hc_head_fn", "hc_head.fn"), ("hc_head_base", "hc_head.base"), ("hc_head_scale", "hc_head.scale"),
    ("embed.weight", "embed_tokens.weight"), ("head.weight", "lm_head.weight"),
)


def rename_v4(name: str) -> str:
    if name == "head.weight":
        return "lm_head.weight"
    if not name.startswith(("model.", "lm_head.")):
        name = "model." + name
    for a, b in _RENAMES:
        if a == "head.weight":
            continue
        name = name.replace(a, b)
    return name


# checkpoint tensors that are stored apart and live in one fused parameter here: (fused, part, which half)
_V4_STACKED = (("compressor.fused_wkv_wgate", "compressor.wkv", 0), ("compressor.fused_wkv_wgate", "compressor.wgate", 1),
               ("attn.fused_wqa_wkv", "attn.wq_a", 0), ("attn.fused_wqa_wkv", "attn.wkv", 1))


class DeepseekV4ForCausalLM(DeepseekV2ForCausalLM):
    def __init__(self, cfg: ModelConfig):
        nn.Module.__init__(self)
        self.cfg = cfg
        self.model = DeepseekV4Model(cfg)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.v4_attention = cfg.compress_ratios is not None
        if self.v4_attention:
            # compressor accumulators are per request and cannot be rebuilt from a cached prefix
            self.supports_prefix_caching = False
            self.allocate_state = self._allocate_state

    # ---- caches of the V4 attention layers ---------------------------------------------------------------------
    def _attn_layers(self):
        return [self.model.layers[str(i)].attn for i in range(self.cfg.num_hidden_layers)]

    def kv_cache_spec(self) -> dict:
        return {"kind": "v4"} if self.v4_attention else super().kv_cache_spec()

    def kv_bytes_per_block(self, block_size: int, kv_cache_dtype: str) -> int:
        if not self.v4_attention:
            return super().kv_bytes_per_block(block_size, kv_cache_dtype)
        elem = torch.empty((), dtype=self.cfg.dtype).element_size()
        return sum(a.bytes_per_block(block_size, elem) for a in self._attn_layers())

    def allocate_kv_cache(self, num_blocks, block_size, kv_cache_dtype, device):
        if not self.v4_attention:
            return super().allocate_kv_cache(num_blocks, block_size, kv_cache_dtype, device)
        if kv_cache_dtype not in ("auto", "bfloat16", "float16", "float32"):
            raise ValueError("the V4 attention path keeps its caches in the model dtype")
        return [a.allocate_kv_cache(num_blocks, block_size, self.cfg.dtype, device) for a in self._attn_layers()]

    def _allocate_state(self, slots: int, device) -> int:
        return sum(a.allocate_state(slots, device) for a in self._attn_layers())

    def _load_v4_attn(self, name: str, w: torch.Tensor, params: dict, modules: dict) -> str:
        """One tensor of a V4 attention block (``layers.N.attn...``) by its release name."""
        if not name.startswith("model."):
            name = "model." + name
        for fused, part, half in _V4_STACKED:
            if f".{part}." in name:
                target = name.replace(part, fused)
                p = params[target]
                off = 0 if half == 0 else p.shape[0] - w.shape[0]
                p.data[off: off + w.shape[0]].copy_(w)
                return target
        p = params[name]
        loader = getattr(modules[name.rsplit(".", 1)[0]], "weight_loader", None)
        if loader is not None:
            loader(p, w, None)
        else:
            p.data.copy_(w.reshape(p.shape))
        return name

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        buffers = dict(self.named_buffers())
        params, modules = dict(self.named_parameters()), dict(self.named_modules())
        direct: set = set()

        def mapped():
            for name, w in weights:
                if self.v4_attention and ".attn." in name:
                    direct.add(self._load_v4_attn(name, w, params, modules))
                    continue
                name = rename_v4(name).replace(".ffn.experts.", ".ffn.experts.").replace(".mlp.", ".ffn.")
                if name.endswith(".tid2eid") and name in buffers:
                    buffers[name].copy_(w.to(torch.int32))
                    continue
                yield name, w

        return super().load_weights(mapped()) | direct


class DeepSeekV4MTP(DeepSeekMTP):
    """V4's MTP heads read the final (head-mixed) hidden state of the target, so the V3 module applies."""
