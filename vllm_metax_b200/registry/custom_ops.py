"""Out-of-tree implementations of vLLM ``CustomOp`` layers on this package's kernels.

One table drives the registration: (upstream module, class name, forward_oot).  Each entry becomes a
subclass of the upstream layer whose ``forward_oot`` calls ``vllm_metax_b200._custom_ops``; vLLM picks it
up through ``CustomOp.register_oot`` when the platform is out-of-tree.
Parity: vllm_metax/registry/custom_ops/activation.py:17-73 (ten activations), layernorm.py:6-20
(RMSNorm, GemmaRMSNorm, RMSNormGated), layers/attention/mm_encoder_attention.py:17-122,
layers/mamba/qwen_gdn_linear_attn.py:16-88, layers/minimax_rms_norm/rms_norm_tp.py:22-59.
"""
from __future__ import annotations

import importlib
from typing import Callable, Optional

import torch

from .. import _custom_ops as ops

REGISTERED: dict[str, type] = {}


def _gated(name: str, **fixed) -> Callable:
    def fwd(self, x: torch.Tensor) -> torch.Tensor:
        p0 = p1 = 0.0
        if name == "fatrelu":
            p0 = float(getattr(self, "threshold", 0.0))
        if name == "swigluoai":
            p0, p1 = float(getattr(self, "alpha", 1.702)), float(getattr(self, "limit", 7.0))
        if name in ("swiglustep", "silu_clamp"):
            p1 = float(getattr(self, "limit", getattr(self, "swiglu_limit", 7.0)))
        return ops.act_and_mul(x, name if name != "silu_clamp" else "swiglustep", p0=p0, p1=p1)

    return fwd


def _plain(name: str) -> Callable:
    def fwd(self, x: torch.Tensor) -> torch.Tensor:
        return ops.activation(x, name)

    return fwd


def _rms_norm(gemma: bool) -> Callable:
    def fwd(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        eps = float(getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6)))
        w = self.weight.data if getattr(self, "has_weight", True) else torch.ones(x.shape[-1], dtype=x.dtype, device=x.device)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if residual is not None:
            r2 = residual.reshape(-1, shape[-1])
            ops.fused_add_rms_norm(x2, r2, w, eps, gemma=gemma)
            return x2.reshape(shape), r2.reshape(shape)
        return ops.rms_norm(x2, w, eps, gemma=gemma).reshape(shape)

    return fwd


def _rms_norm_gated(self, x: torch.Tensor, z: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x) * silu(z) (norm_before_gate) as used by Mamba-2 / gated delta-net blocks."""
    eps = float(getattr(self, "eps", 1e-6))
    if z is not None and not getattr(self, "norm_before_gate", True):
        x = x * torch.nn.functional.silu(z.float()).to(x.dtype)
        z = None
    y = ops.rms_norm(x.reshape(-1, x.shape[-1]), self.weight.data, eps).reshape(x.shape)
    if z is not None:
        y = y * torch.nn.functional.silu(z.float()).to(y.dtype)
    return y


def _mm_encoder_attention(self, query, key, value, cu_seqlens=None, max_seqlen=None, sequence_lengths=None):
    """Vision-encoder attention on the non-causal tcgen05 varlen kernel."""
    from ..layers.mm_encoder_attention import encoder_attention

    hs = self.head_size
    q = query.reshape(*query.shape[:-1], -1, hs) if query.shape[-1] != hs else query
    k = key.reshape(*key.shape[:-1], -1, hs) if key.shape[-1] != hs else key
    v = value.reshape(*value.shape[:-1], -1, hs) if value.shape[-1] != hs else value
    out = encoder_attention(q, k, v, cu_seqlens, None if max_seqlen is None else int(max_seqlen), getattr(self, "scale", None))
    return out.reshape(query.shape) if query.shape[-1] != hs else out


def _chunk_gated_delta_rule(self, q, k, v, g, beta, initial_state, output_final_state, cu_seqlens=None,
                            chunk_indices=None, chunk_offsets=None, use_qk_l2norm_in_kernel=True, core_attn_out=None):
    """GDN prefill on the recurrent kernel: ``q, k [1, T, H, 128]``, ``initial_state [N, Hv, 128, 128]``."""
    from ..ops.gdn import gated_delta_rule

    T = q.shape[-3]
    q3, k3, v3 = (t.reshape(T, t.shape[-2], t.shape[-1]) for t in (q, k, v))
    qsl = cu_seqlens if cu_seqlens is not None else torch.tensor([0, T], dtype=torch.int32, device=q.device)
    n = qsl.numel() - 1
    state = initial_state.float().contiguous() if initial_state is not None else \
        torch.zeros(n, v3.shape[1], q3.shape[-1], v3.shape[-1], dtype=torch.float32, device=q.device)
    idx = torch.arange(n, dtype=torch.int32, device=q.device)
    o = gated_delta_rule(q3, k3, v3, g.reshape(T, -1), beta.reshape(T, -1), qsl, state, idx, None, None,
                         use_qk_l2norm_in_kernel).reshape(v.shape)
    if core_attn_out is not None:
        core_attn_out.copy_(o.reshape(core_attn_out.shape))
        o = core_attn_out
    return o, (state if output_final_state else None)


def _minimax_rms_norm_tp(self, x: torch.Tensor, *args, **kwargs):
    """RMSNorm over a hidden dimension split across the TP ranks: only per-token sums of squares cross NVLink."""
    from ..parallel import state as ps
    from ..parallel.custom_allreduce import CrossRankRMSNorm

    eps = float(getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6)))
    x2 = x.reshape(-1, x.shape[-1])
    if getattr(self, "tp_world", 1) == 1 or not getattr(ps._S, "initialized", False):
        return ops.rms_norm(x2, self.weight.data.to(x.dtype), eps).reshape(x.shape)
    rms = getattr(self, "_b200_rms", None)
    if rms is None or rms.t_cap < x2.shape[0]:
        rms = CrossRankRMSNorm(ps.get_tp_group(), x.device, max(x2.shape[0], 8192))
        self._b200_rms = rms
    return rms(x2.contiguous(), self.weight.data.to(x.dtype), eps)[0].reshape(x.shape)


def _rotary(self, positions: torch.Tensor, query: torch.Tensor, key: Optional[torch.Tensor] = None, *args, **kwargs):
    """RoPE in place on this package's kernel (NeoX or interleaved pairing, partial rotary widths)."""
    offsets = args[0] if args else kwargs.get("offsets")
    if offsets is not None or kwargs.get("inverse", False):
        return self.forward_native(positions, query, key, *args, **kwargs)
    from .c_namespace import fp32_cos_sin

    T = positions.numel()
    q2 = query.view(T, -1)
    k2 = key.view(T, -1) if key is not None else None
    ops.rotary_embedding(positions.reshape(-1), q2, k2, int(self.head_size), fp32_cos_sin(self.cos_sin_cache),
                         bool(self.is_neox_style))
    return query, key


def _rotary_native(self, *args, **kwargs):
    """Multi-axis position schemes (M-RoPE, XD-RoPE) keep upstream's tensor formulation."""
    return self.forward_native(*args, **kwargs)


_TABLE = [
    ("vllm.model_executor.layers.rotary_embedding.base", "RotaryEmbedding", _rotary),
    ("vllm.model_executor.layers.rotary_embedding.llama3_rope", "Llama3RotaryEmbedding", _rotary),
    ("vllm.model_executor.layers.rotary_embedding.linear_scaling_rope", "LinearScalingRotaryEmbedding", _rotary),
    ("vllm.model_executor.layers.rotary_embedding.yarn_scaling_rope", "YaRNScalingRotaryEmbedding", _rotary),
    ("vllm.model_executor.layers.rotary_embedding.deepseek_scaling_rope", "DeepseekScalingRotaryEmbedding", _rotary_native),
    ("vllm.model_executor.layers.rotary_embedding.mrope", "MRotaryEmbedding", _rotary_native),
    ("vllm.model_executor.layers.rotary_embedding.xdrope", "XDRotaryEmbedding", _rotary_native),
    ("vllm.model_executor.layers.activation", "SiluAndMul", _gated("silu")),
    ("vllm.model_executor.layers.activation", "MulAndSilu", _gated("mul_silu")),
    ("vllm.model_executor.layers.activation", "GeluAndMul", None),           # approximate flag read at call
    ("vllm.model_executor.layers.activation", "FatreluAndMul", _gated("fatrelu")),
    ("vllm.model_executor.layers.activation", "SwigluOAIAndMul", _gated("swigluoai")),
    ("vllm.model_executor.layers.activation", "SwigluStepAndMul", _gated("swiglustep")),
    ("vllm.model_executor.layers.activation", "SiluAndMulWithClamp", _gated("silu_clamp")),
    ("vllm.model_executor.layers.activation", "NewGELU", _plain("gelu_new")),
    ("vllm.model_executor.layers.activation", "FastGELU", _plain("gelu_fast")),
    ("vllm.model_executor.layers.activation", "QuickGELU", _plain("gelu_quick")),
    ("vllm.model_executor.layers.layernorm", "RMSNorm", _rms_norm(False)),
    ("vllm.model_executor.layers.layernorm", "GemmaRMSNorm", _rms_norm(True)),
    ("vllm.model_executor.layers.layernorm", "RMSNormGated", _rms_norm_gated),
    ("vllm.model_executor.layers.attention.mm_encoder_attention", "MMEncoderAttention", _mm_encoder_attention),
    ("vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn", "ChunkGatedDeltaRule", _chunk_gated_delta_rule),
    ("vllm.model_executor.layers.mamba.linear_attn", "MiniMaxText01RMSNormTP", _minimax_rms_norm_tp),
]


def _gelu_and_mul(self, x: torch.Tensor) -> torch.Tensor:
    return ops.act_and_mul(x, "gelu_tanh" if getattr(self, "approximate", "none") == "tanh" else "gelu")


def register_all() -> dict[str, type]:
    for mod_name, cls_name, fwd in _TABLE:
        try:
            base = getattr(importlib.import_module(mod_name), cls_name)
        except (ImportError, AttributeError):
            continue
        if cls_name in REGISTERED or not hasattr(base, "register_oot"):
            continue
        impl = fwd if fwd is not None else _gelu_and_mul
        sub = type(f"B200{cls_name}", (base,), {"forward_oot": impl, "__doc__": f"{cls_name} on sm_100a kernels"})
        try:
            base.register_oot(sub)
        except AssertionError:      # another plugin registered this layer first
            continue
        REGISTERED[cls_name] = sub
    return REGISTERED


register_all()
