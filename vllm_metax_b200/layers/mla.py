"""Multi-head latent attention (DeepSeek V2/V3/V3.2) and the V3.2 sparse-attention indexer.

Backends (one kernel each, chosen by what the step contains - not by hardware):

  MLA           latent cache ``[blocks, block_size, 576]`` bf16 (or ``fp8_ds_mla`` 656-byte records)
    prefill without context   -> up-project the latent (kv_b_proj) and run varlen MHA (qk 192 / v 128)
                                 on the tcgen05 prefill kernel
    decode / prefill with context / sparse
                              -> absorbed MQA: q_nope . W_UK, attention over the latent cache
                                 (``mla_decode``), then . W_UV
  MLA_SPARSE    same absorbed kernel restricted to ``topk_indices[t, :]`` from the indexer
  INDEXER       fp8 index keys ``[blocks, block_size*(128+4)]`` (values then f32 scales per block),
                logits ``sum_h w[h] relu(q[h].k) k_scale`` + top-k

Parity: vllm_metax/model_executor/layers/attention/mla_attention.py:588-945 (forward_impl split into
MHA prefill / MQA decode, W_UK_T / W_UV absorption :833-848,1087-1117),
v1/attention/backends/mla/{flashmla,flashmla_sparse,indexer}.py,
registry/custom_ops/layers/sparse_attn_indexer/fp8.py:45-393.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..attention.metadata import get_forward_context


class MLABackend:
    name = "MLA"

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, kv_cache_dtype: str):
        return (num_blocks, block_size, 656 if kv_cache_dtype == "fp8_ds_mla" else 576)

    @staticmethod
    def allocate(num_blocks, block_size, model_dtype, kv_cache_dtype, device):
        if kv_cache_dtype == "fp8_ds_mla":
            return torch.zeros(num_blocks, block_size, 656, dtype=torch.uint8, device=device)
        return torch.zeros(num_blocks, block_size, 576, dtype=model_dtype, device=device)


class IndexerBackend:
    name = "INDEXER"

    @staticmethod
    def allocate(num_blocks, block_size, head_dim, device):
        return torch.zeros(num_blocks, block_size * (head_dim + 4), dtype=torch.uint8, device=device)


class MLAAttention(nn.Module):
    """Attention core given projected q and the new latent entries; owns W_UK / W_UV."""

    def __init__(self, num_heads: int, scale: float, qk_nope: int, qk_rope: int, v_head: int, kv_lora: int,
                 layer_idx: int, dtype=torch.bfloat16):
        super().__init__()
        assert kv_lora == 512 and qk_rope == 64, "latent cache kernels are built for 512 + 64"
        self.num_heads, self.scale = num_heads, scale
        self.qk_nope, self.qk_rope, self.v_head, self.kv_lora = qk_nope, qk_rope, v_head, kv_lora
        self.layer_idx = layer_idx
        # filled by process_weights_after_loading from kv_b_proj
        self.register_buffer("W_UK", torch.zeros(num_heads, qk_nope, kv_lora, dtype=dtype), persistent=False)
        self.register_buffer("W_UV", torch.zeros(num_heads, kv_lora, v_head, dtype=dtype), persistent=False)

    def set_kv_b(self, kv_b_weight: torch.Tensor) -> None:
        """``kv_b_proj.weight [H*(nope+v), kv_lora]`` -> W_UK [H, nope, lora], W_UV [H, lora, v]."""
        w = kv_b_weight.detach().to(self.W_UK.dtype).view(self.num_heads, self.qk_nope + self.v_head, self.kv_lora)
        self.W_UK.copy_(w[:, : self.qk_nope])
        self.W_UV.copy_(w[:, self.qk_nope:].transpose(1, 2))

    def forward(self, q: torch.Tensor, kv_c: torch.Tensor, k_pe: torch.Tensor, kv_b_proj=None,
                topk_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``q [T, H, nope+rope]`` (rope already applied), ``kv_c [T, 512]`` normed, ``k_pe [T, 64]`` roped.
        Returns ``[T, H * v_head]``."""
        ctx = get_forward_context()
        md = ctx.attn_metadata
        cache = ctx.kv_caches[self.layer_idx]["mla"]
        T, H = q.shape[0], self.num_heads
        ops.concat_and_cache_mla(kv_c, k_pe, cache, md.slot_mapping)
        nd, ndt = md.num_decodes, md.num_decode_tokens
        pure_prefill = md.extra.get("prefill_no_context", False) and topk_indices is None and kv_b_proj is not None
        out = torch.empty(T, H, self.v_head, dtype=q.dtype, device=q.device)
        mqa_end = ndt if pure_prefill else T
        if mqa_end > 0:
            n_req = nd if pure_prefill else md.num_reqs
            qa = self._absorb_q(q[:mqa_end])
            lat = ops.mla_decode(qa, cache, md.block_table[:n_req], md.seq_lens[:n_req], self.scale,
                                 query_start_loc=md.query_start_loc[:n_req + 1],
                                 topk_indices=None if topk_indices is None else topk_indices[:mqa_end],
                                 max_seq_len=md.max_seq_len)
            out[:mqa_end] = torch.bmm(lat.transpose(0, 1), self.W_UV).transpose(0, 1)
        if pure_prefill and T > ndt:
            kv = kv_b_proj(kv_c[ndt:]).view(T - ndt, H, self.qk_nope + self.v_head)
            k = torch.cat([kv[..., : self.qk_nope], k_pe[ndt:, None, :].expand(-1, H, -1)], dim=-1).contiguous()
            v = kv[..., self.qk_nope:].contiguous()
            qsl = md.prefill_query_start_loc
            ops.varlen_attention(q[ndt:].contiguous(), k, v, qsl, qsl, self.scale, out=out[ndt:],
                                 max_q_len=md.max_prefill_query_len, causal=True)
        return out.reshape(T, H * self.v_head)

    def _absorb_q(self, q: torch.Tensor) -> torch.Tensor:
        q_nope, q_pe = q[..., : self.qk_nope], q[..., self.qk_nope:]
        ql = torch.bmm(q_nope.transpose(0, 1), self.W_UK).transpose(0, 1)      # [T, H, 512]
        return torch.cat([ql, q_pe], dim=-1).contiguous()


def sparse_attn_indexer(q_fp8: torch.Tensor, weights: torch.Tensor, k: torch.Tensor, idx_cache: torch.Tensor,
                        topk: int, block_size: int) -> torch.Tensor:
    """Insert the new index keys, then top-k cache positions for every new token.

    ``q_fp8 [T, Hi, 128]`` e4m3 values, ``weights [T, Hi]`` (q scale and softmax scale folded in),
    ``k [T, 128]`` (bf16).  Returns int32 ``[T, topk]`` per-request positions, -1 padded.
    """
    md = get_forward_context().attn_metadata
    ops.indexer_k_quant_and_cache(k, idx_cache, md.slot_mapping, block_size)
    return ops.indexer_topk(q_fp8, weights, idx_cache, md.block_table, md.seq_lens, md.query_start_loc, topk,
                            block_size, max_seq_len=md.max_seq_len)
