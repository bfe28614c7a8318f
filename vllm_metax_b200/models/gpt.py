"""LayerNorm + (non-gated) MLP decoders: GPT-NeoX / Pythia, Falcon, BLOOM, MPT, GPT-BigCode (StarCoder), GPT-2.

One graph, described per architecture by a ``GPTSpec``:

    h   = wte[ids] (+ wpe[pos]) (-> LayerNorm for BLOOM)
    per layer
        a = attn(LN1(h))                              fused qkv GEMM -> (RoPE | ALiBi | nothing) + KV write -> paged attention -> dense
        sequential residual:   h = h + a ;  h = h + mlp(LN2(h))
        parallel residual:     h = h + a + mlp(LN2(h) | LN1(h))      (GPT-NeoX, Falcon)
    logits = lm_head(LN_f(h))

Position information is rotary (GPT-NeoX: a fraction of every head; Falcon), ALiBi slopes folded into the attention
kernels (BLOOM, MPT, Falcon-RW), or a learned table (GPT-BigCode, GPT-2).  Checkpoints keep their HF names; the fused
``query_key_value`` tensors come in three layouts (per-head ``[H, 3, D]``, grouped ``[Hkv, q_per_kv + 2, D]``,
concatenated ``q | k | v``) that ``load_weights`` re-orders to ``q | k | v`` before the tensor-parallel split.

Parity: the architectures of the reference's supported-models table that are neither Llama-like nor MoE
(docs/models/supported_models.md:21-47: BloomForCausalLM, FalconForCausalLM, GPTBigCodeForCausalLM,
GPTNeoXForCausalLM, MPTForCausalLM), which the reference serves through upstream model code on its kernels.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Iterable, Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..config import ModelConfig
from ..layers.attention import Attention
from ..layers.basic import LayerNorm, ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.linear import ColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..parallel import state as ps
from ..quantization import get_linear_method


@dataclass
class GPTSpec:
    pos: str = "rope"                    # rope | alibi | learned
    parallel_residual: bool = False
    shared_ln: bool = False              # parallel residual where attention and MLP read the same LayerNorm
    norm_bias: bool = True
    linear_bias: bool = True
    act: str = "gelu"
    emb_ln: bool = False
    qkv_layout: str = "head_interleaved"  # head_interleaved | grouped | concat
    conv1d: bool = False                 # GPT-2: linear weights stored [in, out]
    alibi_scaled: bool = False           # Falcon multiplies the ALiBi bias by 1/sqrt(head_dim) together with the scores
    alibi_bias_max: Optional[float] = None   # MPT slope schedule
    clip_qkv: Optional[float] = None
    renames: list = field(default_factory=list)   # (regex, replacement) applied to checkpoint names in order


def alibi_slopes(num_heads: int, alibi_bias_max: Optional[float] = None) -> torch.Tensor:
    """Per-head slopes.  Default: the geometric schedule of the ALiBi paper with the interleaved extension for head
    counts that are not powers of two (BLOOM, Falcon); with ``alibi_bias_max`` the MPT variant."""
    if alibi_bias_max is not None:
        n2 = 2 ** math.ceil(math.log2(num_heads))
        base = torch.arange(1, n2 + 1, dtype=torch.float32) * (alibi_bias_max / n2)
        s = 1.0 / torch.pow(2.0, base)
        if n2 != num_heads:
            s = torch.cat([s[1::2], s[::2]])[:num_heads]
        return s
    c = 2 ** math.floor(math.log2(num_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(c) - 3)))
    s = torch.pow(torch.tensor(base), torch.arange(1, c + 1, dtype=torch.float32))
    if c != num_heads:
        extra = 2.0 ** (-(2.0 ** -(math.log2(2 * c) - 3)))
        n = min(c, num_heads - c)
        s = torch.cat([s, torch.pow(torch.tensor(extra), torch.arange(1, 1 + 2 * n, 2, dtype=torch.float32))])
    return s


_ACT = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_new", "gelu_fast": "gelu_fast", "gelu": "gelu",
        "bloom_gelu": "gelu_tanh", "relu": "relu", "quick_gelu": "gelu_quick"}


class GPTAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: GPTSpec, layer_idx: int, prefix: str):
        super().__init__()
        tp, rank = ps.tp_size(), ps.tp_rank()
        D = self.head_dim = cfg.head_dim
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, D, cfg.num_attention_heads, cfg.num_key_value_heads,
                                          spec.linear_bias, cfg.dtype, qm("qkv_proj"), prefix=f"{prefix}.qkv_proj")
        self.num_heads, self.num_kv_heads = self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads
        self.q_size, self.kv_size = self.num_heads * D, self.num_kv_heads * D
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * D, cfg.hidden_size, spec.linear_bias, cfg.dtype,
                                        qm("o_proj"), prefix=f"{prefix}.o_proj")
        self.rope, slopes, scale = None, None, D ** -0.5
        if spec.pos == "rope":
            rot = int(D * cfg.partial_rotary_factor)
            self.rope = get_rope(D, rot, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_is_neox, cfg.rope_scaling)
        elif spec.pos == "alibi":
            s = alibi_slopes(cfg.num_attention_heads, spec.alibi_bias_max)
            if spec.alibi_scaled:
                s = s * scale
            slopes = s[rank * self.num_heads: (rank + 1) * self.num_heads].to(torch.float32).contiguous()
            slopes = slopes.to(torch.empty(0).device)
        self.clip = spec.clip_qkv
        self.attn = Attention(self.num_heads, D, scale, self.num_kv_heads, layer_idx, alibi_slopes=slopes)

    def forward(self, positions, h):
        qkv = self.qkv_proj(h)
        if self.clip is not None:
            qkv = qkv.clamp_(-self.clip, self.clip)
        q = qkv[:, : self.q_size]
        k = qkv[:, self.q_size: self.q_size + self.kv_size]
        v = qkv[:, self.q_size + self.kv_size:]
        return self.o_proj(self.attn(q, k, v, positions, self.rope))


class GPTMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: GPTSpec, prefix: str):
        super().__init__()
        qm = lambda name: get_linear_method(cfg, f"{prefix}.{name}")
        self.fc_in = ColumnParallelLinear(cfg.hidden_size, cfg.intermediate_size, spec.linear_bias, cfg.dtype,
                                          qm("fc_in"), prefix=f"{prefix}.fc_in")
        self.fc_out = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, spec.linear_bias, cfg.dtype,
                                        qm("fc_out"), prefix=f"{prefix}.fc_out")
        self.act = _ACT.get(spec.act, spec.act)

    def forward(self, x):
        return self.fc_out(ops.activation(self.fc_in(x), self.act))


class GPTBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: GPTSpec, layer_idx: int, prefix: str):
        super().__init__()
        self.spec = spec
        ln = lambda: LayerNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, bias=spec.norm_bias)
        self.ln_1 = ln()
        self.ln_2 = None if (spec.parallel_residual and spec.shared_ln) else ln()
        self.attn = GPTAttention(cfg, spec, layer_idx, f"{prefix}.attn")
        self.mlp = GPTMLP(cfg, spec, f"{prefix}.mlp")

    def forward(self, positions, h):
        x = self.ln_1(h)
        a = self.attn(positions, x)
        if self.spec.parallel_residual:
            m = self.mlp(x if self.ln_2 is None else self.ln_2(h))
            return h + a + m
        h = h + a
        return h + self.mlp(self.ln_2(h))


class GPTModel(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: GPTSpec, prefix: str = "transformer"):
        super().__init__()
        self.cfg, self.spec = cfg, spec
        pp = ps.get_pp_group()
        n = cfg.num_hidden_layers
        per = (n + pp.world_size - 1) // pp.world_size
        self.start_layer = pp.rank_in_group * per
        self.end_layer = min(n, self.start_layer + per)
        self.wte = self.wpe = self.emb_ln = None
        if pp.is_first_rank:
            self.wte = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
            if spec.pos == "learned":
                self.wpe = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size, dtype=cfg.dtype)
                self.wpe.weight.requires_grad_(False)
            if spec.emb_ln:
                self.emb_ln = LayerNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, bias=spec.norm_bias)
        self.h = nn.ModuleDict({str(i): GPTBlock(cfg, spec, i - self.start_layer, f"{prefix}.h.{i}")
                                for i in range(self.start_layer, self.end_layer)})
        self.ln_f = LayerNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, bias=spec.norm_bias) if pp.is_last_rank else None

    def forward(self, input_ids, positions, intermediate: Optional[dict] = None):
        if self.wte is not None:
            h = self.wte(input_ids)
            if self.wpe is not None:
                h = h + self.wpe(positions)
            if self.emb_ln is not None:
                h = self.emb_ln(h)
        else:
            h = intermediate["hidden_states"]
        for i in range(self.start_layer, self.end_layer):
            h = self.h[str(i)](positions, h)
        if self.ln_f is None:
            return {"hidden_states": h, "residual": None}
        return self.ln_f(h)


class GPTStyleForCausalLM(nn.Module):
    """Engine-facing wrapper; subclasses only provide ``make_spec``."""

    @staticmethod
    def make_spec(cfg: ModelConfig) -> GPTSpec:
        raise NotImplementedError

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.spec = self.make_spec(cfg)
        self.transformer = GPTModel(cfg, self.spec)
        pp = ps.get_pp_group()
        self.lm_head = None
        if pp.is_last_rank:
            if cfg.tie_word_embeddings and self.transformer.wte is not None:
                self.lm_head = self.transformer.wte
                self.lm_head.__class__ = ParallelLMHead
            else:
                self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)

    # ---- engine interface -----------------------------------------------------
    def num_kv_layers(self) -> int:
        return self.transformer.end_layer - self.transformer.start_layer

    def kv_cache_spec(self) -> dict:
        a = next(iter(self.transformer.h.values())).attn
        return {"kind": "gqa", "num_kv_heads": a.num_kv_heads, "head_size": a.head_dim}

    def forward(self, input_ids, positions, intermediate=None):
        return self.transformer(input_ids, positions, intermediate)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head.logits(hidden)

    # ---- weights ----------------------------------------------------------------
    def _qkv_to_concat(self, w: torch.Tensor) -> torch.Tensor:
        """Checkpoint qkv rows (weight ``[rows, in]`` or bias ``[rows]``) -> ``q | k | v`` row order."""
        cfg, lay = self.cfg, self.spec.qkv_layout
        H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        tail = w.shape[1:]
        if lay == "concat" or w.shape[0] != (H + 2 * Hkv) * D:
            return w
        if lay == "head_interleaved":
            if Hkv != H:                          # multi-query checkpoints already store q heads then k, v
                return w
            x = w.reshape(H, 3, D, *tail)
            return torch.cat([x[:, 0].reshape(H * D, *tail), x[:, 1].reshape(H * D, *tail),
                              x[:, 2].reshape(H * D, *tail)], 0)
        g = H // Hkv                              # grouped: every kv head is followed by its q heads' k and v
        x = w.reshape(Hkv, g + 2, D, *tail)
        return torch.cat([x[:, :g].reshape(H * D, *tail), x[:, g].reshape(Hkv * D, *tail),
                          x[:, g + 1].reshape(Hkv * D, *tail)], 0)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded: set[str] = set()
        for name, w in weights:
            for pat, rep in self.spec.renames:
                name = re.sub(pat, rep, name)
            if name.startswith("lm_head.") and self.cfg.tie_word_embeddings:
                continue
            if name not in params:
                continue
            if self.spec.conv1d and w.dim() == 2 and any(s in name for s in ("qkv_proj", "o_proj", "fc_in", "fc_out")):
                w = w.t()
            if ".qkv_proj." in name:
                w = self._qkv_to_concat(w.contiguous())
            p = params[name]
            mod = modules[name.rsplit(".", 1)[0]]
            loader = getattr(mod, "weight_loader", None)
            if loader is not None:
                loader(p, w, None)
            else:
                p.data.copy_(w.reshape(p.shape))
            loaded.add(name)
        for m in self.modules():
            qm = getattr(m, "quant_method", None)
            if qm is not None and hasattr(qm, "process_weights_after_loading"):
                qm.process_weights_after_loading(m)
        return loaded


_BLOOM_NAMES = [(r"^(?!transformer\.|lm_head\.)", "transformer."),          # some exports drop the prefix
                (r"\.word_embeddings\.", ".wte."), (r"\.word_embeddings_layernorm\.", ".emb_ln."),
                (r"\.input_layernorm\.", ".ln_1."), (r"\.post_attention_layernorm\.", ".ln_2."),
                (r"\.self_attention\.query_key_value\.", ".attn.qkv_proj."), (r"\.self_attention\.dense\.", ".attn.o_proj."),
                (r"\.mlp\.dense_h_to_4h\.", ".mlp.fc_in."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.fc_out.")]


class BloomForCausalLM(GPTStyleForCausalLM):
    @staticmethod
    def make_spec(cfg):
        cfg.tie_word_embeddings = cfg.hf_config.get("tie_word_embeddings", True)
        return GPTSpec(pos="alibi", act="gelu_tanh", emb_ln=True, renames=_BLOOM_NAMES)


class FalconForCausalLM(GPTStyleForCausalLM):
    @staticmethod
    def make_spec(cfg):
        hf = cfg.hf_config
        new_arch = bool(hf.get("new_decoder_architecture", False))
        parallel = new_arch or bool(hf.get("parallel_attn", True))
        two_ln = new_arch and (hf.get("num_ln_in_parallel_attn") or 2) == 2
        cfg.tie_word_embeddings = hf.get("tie_word_embeddings", True)
        names = [(r"\.word_embeddings\.", ".wte."),
                 (r"\.ln_attn\.", ".ln_1."), (r"\.ln_mlp\.", ".ln_2."),
                 (r"\.input_layernorm\.", ".ln_1."), (r"\.post_attention_layernorm\.", ".ln_2."),
                 (r"\.self_attention\.query_key_value\.", ".attn.qkv_proj."), (r"\.self_attention\.dense\.", ".attn.o_proj."),
                 (r"\.mlp\.dense_h_to_4h\.", ".mlp.fc_in."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.fc_out.")]
        return GPTSpec(pos="alibi" if hf.get("alibi", False) else "rope", alibi_scaled=True,
                       parallel_residual=parallel, shared_ln=parallel and not two_ln,
                       linear_bias=bool(hf.get("bias", False)), act=hf.get("activation", "gelu"),
                       qkv_layout="grouped" if new_arch else "head_interleaved", renames=names)


class GPTNeoXForCausalLM(GPTStyleForCausalLM):
    @staticmethod
    def make_spec(cfg):
        hf = cfg.hf_config
        if "partial_rotary_factor" not in hf and "rotary_pct" not in hf and not isinstance(hf.get("rope_parameters"), dict):
            cfg.partial_rotary_factor = 0.25
        names = [(r"^gpt_neox\.", "transformer."), (r"^embed_out\.", "lm_head."), (r"\.embed_in\.", ".wte."),
                 (r"\.layers\.", ".h."), (r"\.final_layer_norm\.", ".ln_f."),
                 (r"\.input_layernorm\.", ".ln_1."), (r"\.post_attention_layernorm\.", ".ln_2."),
                 (r"\.attention\.query_key_value\.", ".attn.qkv_proj."), (r"\.attention\.dense\.", ".attn.o_proj."),
                 (r"\.mlp\.dense_h_to_4h\.", ".mlp.fc_in."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.fc_out.")]
        return GPTSpec(pos="rope", parallel_residual=bool(hf.get("use_parallel_residual", True)),
                       linear_bias=bool(hf.get("attention_bias", True)), act=hf.get("hidden_act", "gelu"), renames=names)


class MPTForCausalLM(GPTStyleForCausalLM):
    @staticmethod
    def make_spec(cfg):
        hf = cfg.hf_config
        ac = hf.get("attn_config") or {}
        assert not ac.get("qk_ln", False), "MPT qk_ln is not supported"
        cfg.tie_word_embeddings = hf.get("tie_word_embeddings", True)
        names = [(r"\.blocks\.", ".h."), (r"\.norm_1\.", ".ln_1."), (r"\.norm_2\.", ".ln_2."), (r"\.norm_f\.", ".ln_f."),
                 (r"\.attn\.Wqkv\.", ".attn.qkv_proj."), (r"\.attn\.out_proj\.", ".attn.o_proj."),
                 (r"\.ffn\.up_proj\.", ".mlp.fc_in."), (r"\.ffn\.down_proj\.", ".mlp.fc_out.")]
        no_bias = bool(hf.get("no_bias", True))
        return GPTSpec(pos="alibi" if ac.get("alibi", True) else "learned", alibi_bias_max=float(ac.get("alibi_bias_max", 8)),
                       clip_qkv=ac.get("clip_qkv"), norm_bias=not no_bias, linear_bias=not no_bias, act="gelu",
                       qkv_layout="concat", renames=names)


class GPTBigCodeForCausalLM(GPTStyleForCausalLM):
    conv1d = False

    @classmethod
    def make_spec(cls, cfg):
        hf = cfg.hf_config
        cfg.tie_word_embeddings = hf.get("tie_word_embeddings", True)
        names = [(r"\.attn\.c_attn\.", ".attn.qkv_proj."), (r"\.attn\.c_proj\.", ".attn.o_proj."),
                 (r"\.mlp\.c_fc\.", ".mlp.fc_in."), (r"\.mlp\.c_proj\.", ".mlp.fc_out.")]
        return GPTSpec(pos="learned", act=hf.get("activation_function", "gelu_pytorch_tanh"), conv1d=cls.conv1d,
                       qkv_layout="concat" if cls.conv1d else "head_interleaved", renames=names)


class GPT2LMHeadModel(GPTBigCodeForCausalLM):
    conv1d = True
