"""Configuration objects of the standalone engine.

``ModelConfig`` mirrors the fields of a HuggingFace ``config.json`` that the
model classes read (Llama / Qwen3 / Qwen3-MoE / DeepSeek-V2/V3/V3.2), so a
checkpoint directory and a hand-written dict are interchangeable.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "float16": torch.float16, "half": torch.float16,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "auto": None}


def resolve_dtype(d) -> Optional[torch.dtype]:
    if isinstance(d, torch.dtype) or d is None:
        return d
    return _DTYPES[str(d)]


def _canonical_hf_keys(d: dict) -> dict:
    """Copy of a HF ``config.json`` dict with the spellings older / non-Llama architectures use mapped onto the
    Llama-style keys the rest of the parser reads (GPT-2 era ``n_embd`` / ``n_head`` / ``n_layer``, MPT ``d_model``,
    Falcon / BigCode multi-query flags, ``rope_parameters`` of recent transformers releases)."""
    d = dict(d)

    def alias(key, *others):
        if d.get(key) is None:
            for o in others:
                if d.get(o) is not None:
                    d[key] = d[o]
                    return

    arch = (d.get("architectures") or [""])[0]
    alias("hidden_size", "n_embd", "d_model")
    alias("num_attention_heads", "n_head", "n_heads")
    if d.get("num_attention_heads") is None and d.get("model_type") == "mamba":
        d["num_attention_heads"] = 1                          # attention-free
    alias("num_hidden_layers", "n_layer", "n_layers", "num_layers")
    alias("rms_norm_eps", "layer_norm_eps", "layer_norm_epsilon", "layernorm_epsilon")
    alias("max_position_embeddings", "n_positions", "max_seq_len", "seq_length")
    alias("intermediate_size", "ffn_hidden_size", "n_inner")
    if d.get("intermediate_size") is None and d.get("expansion_ratio") and d.get("hidden_size"):
        d["intermediate_size"] = int(d["expansion_ratio"] * d["hidden_size"])
    rp = d.get("rope_parameters")
    if isinstance(rp, dict):
        if d.get("rope_theta") is None and rp.get("rope_theta") is not None:
            d["rope_theta"] = rp["rope_theta"]
        if d.get("rope_scaling") is None and rp.get("rope_type", "default") not in (None, "default"):
            d["rope_scaling"] = rp
        if d.get("partial_rotary_factor") is None and rp.get("partial_rotary_factor") is not None:
            d["partial_rotary_factor"] = rp["partial_rotary_factor"]
    alias("head_dim", "kv_channels")
    alias("num_experts", "moe_num_experts")                    # Ernie-4.5-MoE spellings
    alias("num_experts_per_tok", "moe_k")
    alias("n_shared_experts", "moe_num_shared_experts")
    alias("first_k_dense_replace", "moe_layer_start_index")
    alias("moe_layer_freq", "moe_layer_interval")
    if "ChatGLM" in arch and d.get("padded_vocab_size"):
        d["vocab_size"] = d["padded_vocab_size"]
    alias("vocab_size", "padded_vocab_size")
    alias("rope_theta", "rotary_emb_base")
    alias("partial_rotary_factor", "rotary_pct")
    if d.get("num_key_value_heads") is None:
        if "Falcon" in arch:
            if d.get("new_decoder_architecture"):
                d["num_key_value_heads"] = d.get("num_kv_heads") or d.get("num_attention_heads")
            elif d.get("multi_query", True):
                d["num_key_value_heads"] = 1
        elif "GPTBigCode" in arch and d.get("multi_query", True):
            d["num_key_value_heads"] = 1
        elif d.get("multi_query_group_num") is not None and d.get("multi_query_attention", True):
            d["num_key_value_heads"] = d["multi_query_group_num"]
    return d


_DEEPSEEK_V3_MODEL_TYPES = ("joyai_llm_flash", "kimi_k2", "AXK1", "pangu_ultra_moe", "glm4_moe_lite", "longcat_flash",
                            "deepseek_v3", "deepseek_v2")


@dataclass
class ModelConfig:
    architecture: str = "LlamaForCausalLM"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    attention_out_bias: bool = False           # bias on o_proj too (Llama-style ``attention_bias``, InternLM ``bias``)
    qk_norm: bool = False                      # Qwen3: per-head RMSNorm on q and k
    sliding_window: Optional[int] = None
    # ---- MoE -----------------------------------------------------------
    num_experts: int = 0                       # routed experts (0 = dense)
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    n_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0   # Qwen2-MoE: one gated shared expert of this width (0: n_shared * moe width)
    decoder_sparse_step: int = 1               # Qwen MoE: layer i is sparse when (i + 1) % step == 0 ...
    mlp_only_layers: tuple = ()                # ... and i is not listed here
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    scoring_func: str = "softmax"              # softmax | sigmoid | sqrtsoftplus
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    topk_method: str = "greedy"                # greedy | noaux_tc | group_limited_greedy
    # ---- MLA (DeepSeek) -------------------------------------------------
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # ---- DSA indexer (DeepSeek-V3.2) --------------------------------------
    index_n_heads: int = 0
    index_head_dim: int = 128
    index_topk: int = 0
    # ---- MTP ----------------------------------------------------------------
    num_nextn_predict_layers: int = 0
    # ---- DeepSeek-V4 hyper-connections / hash routing -------------------------
    hc_mult: int = 0                           # residual streams (0 = plain residual)
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    num_hash_layers: int = 0                   # leading MoE layers routed by token id (tid2eid table)
    # ---- DeepSeek-V4 attention: one shared 512-wide K = V vector per token, a sliding window of raw vectors plus a
    # ratio-c compressed cache (per layer: 0 / 1 = window only, 4 = compressed + top-k indexer, 128 = compressed, dense)
    compress_ratios: Optional[list] = None     # None = V3.2-style latent attention without compression
    o_lora_rank: int = 0                       # grouped low-rank output projection (wo_a / wo_b)
    o_groups: int = 1
    # ---- numerics / quantisation ----------------------------------------
    dtype: torch.dtype = torch.bfloat16
    quantization: Optional[str] = None         # None | fp8 | w8a8_int8 | awq | gptq | ...
    quant_config: dict = field(default_factory=dict)
    model_path: Optional[str] = None
    seed: int = 0
    # multi-LoRA serving (lora/): slots resident at once and the largest adapter rank
    enable_lora: bool = False
    max_loras: int = 4
    max_lora_rank: int = 64
    eos_token_id: Optional[int] = None
    partial_rotary_factor: float = 1.0         # fraction of each head that is rotated (GPT-NeoX, GLM: < 1)
    use_alibi: bool = False                    # ALiBi slopes instead of rotary embeddings (Baichuan 13B)
    rope_is_neox: bool = True                  # False: GPT-J style (adjacent pairs), e.g. GLM / ChatGLM
    hf_config: dict = field(default_factory=dict, repr=False)   # raw config.json for architecture-specific keys

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        self.dtype = resolve_dtype(self.dtype) or torch.bfloat16

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def has_indexer(self) -> bool:
        return self.index_topk > 0

    def layer_is_moe(self, i: int) -> bool:
        if not self.is_moe or i in self.mlp_only_layers or (i + 1) % max(self.decoder_sparse_step, 1) != 0:
            return False
        return i >= self.first_k_dense_replace and (i % max(self.moe_layer_freq, 1) == 0)

    @classmethod
    def from_hf_dict(cls, d: dict, **overrides: Any) -> "ModelConfig":
        raw = d
        if isinstance(d.get("llm_config"), dict) and "text_config" not in d:      # InternVL's original export
            d = dict(d, text_config=d["llm_config"])
            raw = d
        if isinstance(d.get("text_config"), dict):     # vision-language wrappers: the decoder's fields live one level down
            d = dict(d["text_config"], architectures=d.get("architectures"),
                     **{k: d[k] for k in ("quantization_config", "torch_dtype", "dtype") if k in d and k not in d["text_config"]})
        d = _canonical_hf_keys(d)
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        arch = archs[0]
        # checkpoints that are the DeepSeek-V3 graph (MLA + routed experts) under an architecture name of their own:
        # served by that model class (the reference marks the same model types as MLA models,
        # vllm_metax/patch/enhancement/joyai_support/model_arch_config_convertor.py:22-47)
        from .models import _MODELS

        if arch not in _MODELS and d.get("kv_lora_rank") is not None and \
                d.get("model_type") in _DEEPSEEK_V3_MODEL_TYPES:
            arch = "DeepseekV3ForCausalLM"
        # DeepSeek-V3 lineage: sigmoid scores + bias-corrected grouped top-k even when the config (HF-native exports)
        # does not spell it out
        # (vision-language wrappers follow the rules of their decoder)
        rule_arch = {"Glm4vMoeForConditionalGeneration": "Glm4MoeForCausalLM"}.get(arch, arch)
        v3_routing = any(t in rule_arch for t in ("DeepseekV3", "DeepseekV32", "GlmMoeDsa", "DeepseekV4", "Glm4Moe"))
        kw: dict[str, Any] = dict(
            hf_config=dict(raw),
            partial_rotary_factor=float(d.get("partial_rotary_factor", 1.0) or 1.0),
            rope_is_neox=bool(d.get("rope_is_neox", True)),
            architecture=arch,
            vocab_size=d.get("vocab_size", 32000),
            hidden_size=d["hidden_size"],
            intermediate_size=d.get("intermediate_size", 4 * d["hidden_size"]),
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads"),
            head_dim=d.get("head_dim"),
            rms_norm_eps=d.get("rms_norm_eps", 1e-5),
            rope_theta=d.get("rope_theta", 10000.0),
            rope_scaling=d.get("rope_scaling"),
            max_position_embeddings=d.get("max_position_embeddings", 8192),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            hidden_act=d.get("hidden_act", "silu"),
            attention_bias=bool(d.get("attention_bias", False) or d.get("bias", False) or d.get("add_qkv_bias", False)
                                or d.get("qkv_bias", False) or ("Qwen2" in arch) or arch == "QWenLMHeadModel"
                                or d.get("model_type") == "qwen2"),
            attention_out_bias=bool((d.get("attention_bias", False) and "Qwen" not in arch and "Glm" not in arch
                                     and "GLM" not in arch) or (d.get("bias", False) and "InternLM" in arch)),
            mlp_bias=d.get("mlp_bias", False),
            qk_norm=("Qwen3" in arch) or bool(d.get("use_qk_norm", False)),
            sliding_window=d.get("sliding_window") if d.get("use_sliding_window", True) else None,
            num_experts=d.get("num_experts", d.get("n_routed_experts", d.get("num_local_experts", 0))) or 0,
            num_experts_per_tok=d.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=d.get("moe_intermediate_size") or d.get("intermediate_size", 0) or 0,
            shared_expert_intermediate_size=d.get("shared_expert_intermediate_size", 0) or 0,
            decoder_sparse_step=d.get("decoder_sparse_step", 1) or 1,
            mlp_only_layers=tuple(d.get("mlp_only_layers") or ()),
            norm_topk_prob=d.get("norm_topk_prob", True),
            n_shared_experts=d.get("n_shared_experts", 0) or (1 if d.get("shared_expert_intermediate_size") else 0),
            first_k_dense_replace=d.get("first_k_dense_replace", 0) or 0,
            moe_layer_freq=d.get("moe_layer_freq", 1) or 1,
            scoring_func=d.get("scoring_func", "sigmoid" if v3_routing else "softmax"),
            n_group=d.get("n_group", 1) or 1,
            topk_group=d.get("topk_group", 1) or 1,
            routed_scaling_factor=d.get("routed_scaling_factor", 1.0) or 1.0,
            topk_method=d.get("topk_method", "noaux_tc" if v3_routing else "greedy"),
            q_lora_rank=d.get("q_lora_rank"),
            kv_lora_rank=d.get("kv_lora_rank", 0) or 0,
            qk_nope_head_dim=d.get("qk_nope_head_dim", 0) or 0,
            qk_rope_head_dim=d.get("qk_rope_head_dim", 0) or 0,
            v_head_dim=d.get("v_head_dim", 0) or 0,
            index_n_heads=d.get("index_n_heads", 0) or 0,
            index_head_dim=d.get("index_head_dim", 128) or 128,
            index_topk=d.get("index_topk", 0) or 0,
            num_nextn_predict_layers=d.get("num_nextn_predict_layers", 0) or 0,
            hc_mult=d.get("hc_mult", 0) or 0, hc_sinkhorn_iters=d.get("hc_sinkhorn_iters", 20) or 20,
            hc_eps=d.get("hc_eps", 1e-6) or 1e-6, num_hash_layers=d.get("num_hash_layers", 0) or 0,
            compress_ratios=d.get("compress_ratios"), o_lora_rank=d.get("o_lora_rank", 0) or 0,
            o_groups=d.get("o_groups", 1) or 1,
            dtype=d.get("torch_dtype", d.get("dtype", "bfloat16")),
            eos_token_id=(d.get("eos_token_id")[0] if isinstance(d.get("eos_token_id"), list) else d.get("eos_token_id")),
        )
        qc = d.get("quantization_config")
        if qc:
            kw["quantization"] = qc.get("quant_method")
            kw["quant_config"] = qc
        kw.update(overrides)
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str, **overrides: Any) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        return cls.from_hf_dict(d, model_path=path, **overrides)


@dataclass
class CacheConfig:
    block_size: int = 64
    num_gpu_blocks: Optional[int] = None       # None: derived from gpu_memory_utilization
    gpu_memory_utilization: float = 0.88
    kv_cache_dtype: str = "auto"               # auto | bfloat16 | float16 | fp8 | int8_per_token_head | fp8_per_token_head | fp8_ds_mla | turboquant_{k8v4,4bit_nc,k3v4_nc,3bit_nc}
    enable_prefix_caching: bool = False      # (pre-empted requests are recomputed; there is no CPU swap space)


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    # accepted for command-line compatibility: the experts of a MoE model are always sharded over the ranks of the
    # tensor-parallel group (and over all replicas with data_parallel_size > 1)
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    prefill_context_parallel_size: int = 1
    # sequence-parallel MoE inside one replica: every rank routes 1 / tp of the tokens and the rows are exchanged
    # (layers/fused_moe.py:_forward_sp) instead of every rank running its experts on all tokens; the exchange runs
    # over the NVLink dispatch / combine kernels ("fused_nvlink") or all-gather / reduce-scatter collectives
    use_sequence_parallel_moe: bool = False
    all2all_backend: str = "fused_nvlink"      # fused_nvlink | allgather_reducescatter
    # expert-parallel load balancing (parallel/eplb.py): redundant expert slots, re-placement every
    # eplb_step_interval engine steps from the routing statistics of the last eplb_window steps
    enable_eplb: bool = False
    num_redundant_experts: int = 0
    eplb_step_interval: int = 3000
    eplb_window: int = 1000
    eplb_log_balancedness: bool = False

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size * self.pipeline_parallel_size


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    enable_chunked_prefill: bool = True
    # "fcfs": arrival order.  "priority": a smaller ``priority`` value is admitted first (ties by arrival) and is
    # pre-empted last.
    policy: str = "fcfs"


@dataclass
class EngineConfig:
    model: ModelConfig
    cache: CacheConfig = field(default_factory=CacheConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    device: str = "cuda"
    enforce_eager: bool = False
    load_format: str = "auto"                  # auto | dummy | safetensors | sharded_state
    additional_config: dict = field(default_factory=dict)
