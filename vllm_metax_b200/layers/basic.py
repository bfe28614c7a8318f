"""Norms, embeddings, rotary embedding, activations as ``nn.Module``s over ``_custom_ops``.

Parity: vllm_metax/registry/custom_ops/{layernorm,activation}.py and
layers/rotary_embedding/rotary_embedding.py redirect the upstream CustomOp classes
to their CUDA path on the out-of-tree platform; here the modules call the sm_100a
kernels directly.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..ops import reference as ref
from ..parallel import state as ps


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.bfloat16, gemma: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.eps = eps
        self.gemma = gemma

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """Without residual: returns norm(x).  With residual: in place ``residual += x; x = norm(residual)``
        and returns ``(x, residual)``."""
        if residual is None:
            return ops.rms_norm(x, self.weight, self.eps, gemma=self.gemma)
        return ops.fused_add_rms_norm(x, residual, self.weight, self.eps, gemma=self.gemma)


class GemmaRMSNorm(RMSNorm):
    def __init__(self, hidden_size, eps=1e-6, dtype=torch.bfloat16):
        super().__init__(hidden_size, eps, dtype, gemma=True)
        self.weight.data.zero_()


class RMSNormGated(nn.Module):
    def __init__(self, hidden_size, eps=1e-6, dtype=torch.bfloat16):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x, gate):
        y = ops.rms_norm(x, self.weight, self.eps)
        return (y.float() * torch.nn.functional.silu(gate.float())).to(x.dtype)


class LayerNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-6, dtype=torch.bfloat16, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype), requires_grad=False) if bias else None
        self.eps = eps

    def forward(self, x):
        return ref.layer_norm(x, self.weight, self.bias, self.eps)


class SiluAndMul(nn.Module):
    def forward(self, x):
        return ops.silu_and_mul(x)


class ActAndMul(nn.Module):
    def __init__(self, act: str = "silu"):
        super().__init__()
        self.act = {"gelu_pytorch_tanh": "gelu_tanh"}.get(act, act)

    def forward(self, x):
        return ops.act_and_mul(x, self.act)


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded over the vocabulary; out-of-shard ids contribute zeros and the
    partial lookups are summed over the TP group."""

    def __init__(self, vocab_size: int, hidden_size: int, dtype=torch.bfloat16):
        super().__init__()
        self.tp = ps.tp_size()
        self.vocab_size = vocab_size
        self.padded = (vocab_size + 64 * self.tp - 1) // (64 * self.tp) * (64 * self.tp)
        self.per = self.padded // self.tp
        self.start = ps.tp_rank() * self.per
        self.weight = nn.Parameter(torch.zeros(self.per, hidden_size, dtype=dtype), requires_grad=False)

    def weight_loader(self, param, loaded, shard_id=None):
        end = min(self.start + self.per, loaded.shape[0])
        if end > self.start:
            param.data[: end - self.start].copy_(loaded[self.start:end])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        y = ops.embedding(self.weight, ids.reshape(-1), vocab_start=self.start)
        if self.tp > 1:
            y = ps.tensor_model_parallel_all_reduce(y)
        return y


class ParallelLMHead(VocabParallelEmbedding):
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        y = ops.gemm(hidden, self.weight)
        if self.tp > 1:
            y = ps.tensor_model_parallel_all_gather(y, -1)
        return y[:, : self.vocab_size]


class RotaryEmbedding(nn.Module):
    """cos/sin table (f32) + the fused RoPE kernel.  ``rope_scaling`` follows HF config dicts
    (linear, llama3, yarn, deepseek_yarn)."""

    def __init__(self, head_size: int, rotary_dim: int, max_position: int, base: float, is_neox: bool = True,
                 rope_scaling: Optional[dict] = None):
        super().__init__()
        self.head_size, self.rotary_dim, self.is_neox = head_size, rotary_dim, is_neox
        cache = ref.build_rope_cache(rotary_dim, max_position, base, torch.float32, rope_scaling)
        self.register_buffer("cos_sin_cache", cache, persistent=False)

    def forward(self, positions, q, k=None):
        return ops.rotary_embedding(positions, q, k, self.head_size, self.cos_sin_cache, self.is_neox)


_ROPE_CACHE: dict = {}


def get_rope(head_size, rotary_dim, max_position, base, is_neox=True, rope_scaling=None) -> RotaryEmbedding:
    key = (head_size, rotary_dim, max_position, base, is_neox, str(rope_scaling), str(torch.get_default_device()))
    if key not in _ROPE_CACHE:
        _ROPE_CACHE[key] = RotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox, rope_scaling)
    return _ROPE_CACHE[key]
