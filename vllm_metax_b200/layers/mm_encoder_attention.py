"""Bidirectional attention over packed image / audio patches (vision-transformer encoders of multimodal models).

``MMEncoderAttention(q, k, v, cu_seqlens, max_seqlen)`` takes ``[T, H, D]`` (or ``[B, S, H, D]``) tensors whose
sequences - one per image or per window - are delimited by ``cu_seqlens`` and runs the non-causal path of the
tcgen05 varlen attention kernel (``csrc/attn_prefill_tcgen05.cu``); on CPU the fp32 statement is used.
Parity: vllm_metax/registry/custom_ops/layers/attention/mm_encoder_attention.py:17-122 and the
``maca_flash_attn_maxseqlen_wrapper`` op of v1/attention/ops/vit_attn_wrappers.py:26-109.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops


def encoder_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None,
                      max_seqlen: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    batched = q.dim() == 4
    if batched:
        B, S = q.shape[:2]
        q, k, v = (t.reshape(B * S, t.shape[2], t.shape[3]) for t in (q, k, v))
        if cu_seqlens is None:
            cu_seqlens = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
            max_seqlen = S
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
    cu = cu_seqlens.int()
    if max_seqlen is None:
        max_seqlen = int((cu[1:] - cu[:-1]).max())
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    out = ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, scale, max_q_len=int(max_seqlen),
                               causal=False)
    return out.reshape(B, S, out.shape[1], out.shape[2]) if batched else out


class MMEncoderAttention(nn.Module):
    def __init__(self, num_heads: int, head_size: int, scale: Optional[float] = None, num_kv_heads: Optional[int] = None):
        super().__init__()
        self.num_heads, self.head_size = num_heads, head_size
        self.num_kv_heads = num_kv_heads or num_heads
        self.scale = head_size ** -0.5 if scale is None else scale

    def forward(self, query, key, value, cu_seqlens=None, max_seqlen=None, sequence_lengths=None):
        def heads(t, n):                     # [..., n * head_size] -> [..., n, head_size]
            flat = t.shape[-1] == n * self.head_size and (n > 1 or t.dim() == 2)
            return t.reshape(*t.shape[:-1], n, self.head_size) if flat else t

        q, k, v = heads(query, self.num_heads), heads(key, self.num_kv_heads), heads(value, self.num_kv_heads)
        ms = None if max_seqlen is None else int(max_seqlen)
        return encoder_attention(q, k, v, cu_seqlens, ms, self.scale)
