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
        pcp_slots = md.extra.get("pcp_slots_all")
        if pcp_slots is not None:
            # prefill context parallel: this copy computed a slice of every chunk; the copies exchange their latent
            # rows and each writes all of them into its own (replicated) cache, after which the slice is an ordinary
            # request of length "end of the slice" for the kernels below - parallel/pcp.py
            from ..parallel import state as ps

            g, sizes = ps.get_pcp_group(), md.extra["pcp_sizes"]
            ops.concat_and_cache_mla(g.all_gatherv(kv_c.contiguous(), sizes), g.all_gatherv(k_pe.contiguous(), sizes),
                                     cache, pcp_slots)
        else:
            ops.concat_and_cache_mla(kv_c, k_pe, cache, md.slot_mapping)
        if "dcp_ctx_lens" in md.extra:
            return self._forward_dcp(q, kv_c, k_pe, kv_b_proj, topk_indices, md, cache)
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

    def _forward_dcp(self, q, kv_c, k_pe, kv_b_proj, topk_indices, md, cache) -> torch.Tensor:
        """Decode context parallel: the latent cache of a sequence is spread over the DCP group (position p on rank
        p % dcp, the slot mapping is -1 elsewhere).  The absorbed queries of all the group's heads are gathered, every
        rank attends its shard, and the partial outputs are combined by their log-sum-exp and scattered back over
        heads (``parallel/dcp.py``).  A step with multi-token requests treats every token as a request of its own
        whose length is the number of local entries it may see, which makes the causal mask exact on an interleaved
        shard; ``topk_indices`` (global positions from the DCP indexer) are reduced to the local ones.
        Mirrors vllm_metax/model_executor/layers/attention/mla_attention.py:858-899, 2142-2297."""
        from ..parallel import dcp
        from ..parallel import state as ps

        g = ps.get_dcp_group()
        d, r = g.world_size, g.rank_in_group
        T, H = q.shape[0], self.num_heads
        nd, ndt = md.num_decodes, md.num_decode_tokens
        pure_prefill = md.extra.get("prefill_no_context", False) and topk_indices is None and kv_b_proj is not None
        out = torch.empty(T, H, self.v_head, dtype=q.dtype, device=q.device)
        mqa_end = ndt if pure_prefill else T
        if mqa_end > 0:
            if "dcp_vis_lens" in md.extra:
                lens = md.extra["dcp_vis_lens"][:mqa_end]
                table = md.block_table[md.extra["dcp_token_req"][:mqa_end]]
            else:                                   # one token per request
                lens, table = md.seq_lens[:mqa_end], md.block_table[:mqa_end]
            local_idx = None
            if topk_indices is not None:
                ti = topk_indices[:mqa_end]
                local_idx = torch.where((ti >= 0) & (ti % d == r), ti // d, torch.full_like(ti, -1)).contiguous()
                empty = (local_idx >= 0).sum(1) == 0
            else:
                empty = lens == 0
            qa = self._absorb_q(q[:mqa_end])

            def attend(q_all):
                lse = torch.empty(H * d, mqa_end, dtype=torch.float32, device=q.device)
                o = ops.mla_decode(q_all, cache, table, lens.clamp_min(1), self.scale, topk_indices=local_idx,
                                   lse_out=lse, max_seq_len=md.max_seq_len)
                lse = torch.where(empty[None, :], torch.full_like(lse, float("-inf")), lse)
                return torch.where(empty[:, None, None], torch.zeros_like(o), o), lse.t().contiguous()

            lat = dcp.decode_attention(qa, attend, g)
            out[:mqa_end] = torch.bmm(lat.transpose(0, 1), self.W_UV).transpose(0, 1)
        if pure_prefill and T > ndt:               # fresh chunks see only their own keys: no communication
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
    pcp_slots = md.extra.get("pcp_slots_all")
    if pcp_slots is not None:       # prefill context parallel: the index keys of all copies go into every copy's cache
        from ..parallel import state as ps

        k_all = ps.get_pcp_group().all_gatherv(k.contiguous(), md.extra["pcp_sizes"])
        ops.indexer_k_quant_and_cache(k_all, idx_cache, pcp_slots, block_size)
    else:
        ops.indexer_k_quant_and_cache(k, idx_cache, md.slot_mapping, block_size)
    if "dcp_ctx_lens" in md.extra:
        return _sparse_attn_indexer_dcp(q_fp8, weights, idx_cache, topk, block_size, md)
    return ops.indexer_topk(q_fp8, weights, idx_cache, md.block_table, md.seq_lens, md.query_start_loc, topk,
                            block_size, max_seq_len=md.max_seq_len)


def _sparse_attn_indexer_dcp(q_fp8, weights, idx_cache, topk: int, block_size: int, md) -> torch.Tensor:
    """Indexer under decode context parallelism: every rank scores the index keys of its shard (token = request, length
    = visible local entries), keeps its top-k with their logits, and the group's candidates are merged into the global
    top-k.  Returns GLOBAL positions.  Mirrors registry/custom_ops/layers/sparse_attn_indexer/fp8.py:241-249."""
    from ..parallel import state as ps

    g = ps.get_dcp_group()
    d, r = g.world_size, g.rank_in_group
    T = q_fp8.shape[0]
    if "dcp_vis_lens" in md.extra:
        lens = md.extra["dcp_vis_lens"][:T]
        table = md.block_table[md.extra["dcp_token_req"][:T]]
    else:
        lens, table = md.seq_lens[:T], md.block_table[:T]
    qsl = torch.arange(T + 1, dtype=torch.int32, device=q_fp8.device)
    local_max = (md.max_seq_len + d - 1) // d
    idx, logits = ops.indexer_topk(q_fp8, weights, idx_cache, table, lens.clamp_min(1), qsl, topk, block_size,
                                   max_seq_len=local_max, return_logits=True)
    ok = (idx >= 0) & (lens > 0)[:, None]
    vals = torch.where(ok, logits.gather(1, idx.clamp_min(0).long()), torch.full_like(idx, float("-inf"), dtype=torch.float32))
    pos = torch.where(ok, idx * d + r, torch.full_like(idx, -1))
    all_vals = g.all_gather(vals.contiguous(), 1)                 # [T, d * topk]
    all_pos = g.all_gather(pos.contiguous(), 1)
    top = torch.topk(all_vals, topk, dim=1)
    sel = all_pos.gather(1, top.indices)
    return torch.where(torch.isfinite(top.values), sel, torch.full_like(sel, -1)).to(torch.int32).contiguous()
