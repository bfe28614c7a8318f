"""The GQA attention layer: fused RoPE + KV-cache write, then the split forward
(decode slice -> split-KV decode kernel, prefill slice -> tcgen05 varlen kernel).

One backend (``PAGED_GQA``) replaces the reference's FLASH_ATTN / TRITON_ATTN /
FLASHINFER family for decoder self-attention: bf16/fp16 caches, fp8 caches with a
static scale, and int8 / fp8 caches with per-(token, head) scales
(``int8_per_token_head``) all run through the same two kernels.  The split of a
mixed batch into a decode slice and a prefill slice follows
vllm_metax/v1/attention/backends/flash_attn.py:1302-1355 (VLLM_METAX_ENABLE_FA_SPLIT_FORWARD).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..attention.metadata import get_forward_context
from ..ops import turboquant as tq

KV_DTYPES = {
    "auto": None, "bfloat16": torch.bfloat16, "float16": torch.float16, "fp8": torch.float8_e4m3fn,
    "fp8_e4m3": torch.float8_e4m3fn, "int8_per_token_head": torch.int8, "fp8_per_token_head": torch.float8_e4m3fn,
}


class PagedGQABackend:
    name = "PAGED_GQA"
    supported_head_sizes = (64, 128, 256)
    supported_kv_cache_dtypes = tuple(KV_DTYPES)

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int):
        return (num_blocks, 2, block_size, num_kv_heads, head_size)

    @staticmethod
    def get_scale_shape(num_blocks: int, block_size: int, num_kv_heads: int):
        return (num_blocks, 2, block_size, num_kv_heads)

    @staticmethod
    def supported_block_sizes():
        return (16, 32, 64, 128, 256)

    @staticmethod
    def allocate(num_blocks, block_size, num_kv_heads, head_size, model_dtype, kv_cache_dtype: str, device):
        if tq.is_turboquant(kv_cache_dtype):
            # combined K+V slots; the second element carries the format instead of a scale tensor
            assert head_size == tq.D, "TurboQuant caches are built for head_dim 128"
            fmt = tq.TqFormat.from_name(kv_cache_dtype)
            return (tq.alloc_cache(num_blocks, block_size, num_kv_heads, fmt, device), fmt)
        dt = KV_DTYPES[kv_cache_dtype] or model_dtype
        cache = torch.zeros(PagedGQABackend.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size),
                            dtype=dt, device=device)
        scales = None
        if kv_cache_dtype.endswith("per_token_head"):
            scales = torch.ones(PagedGQABackend.get_scale_shape(num_blocks, block_size, num_kv_heads),
                                dtype=torch.float32, device=device)
        return (cache, scales)


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int, layer_idx: int,
                 sliding_window: Optional[int] = None, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                 k_scale: float = 1.0, v_scale: float = 1.0, alibi_slopes: Optional[torch.Tensor] = None):
        super().__init__()
        self.alibi_slopes = alibi_slopes           # f32 [num_heads] (Bloom / MPT / Baichuan-13B style position bias)
        self.num_heads, self.head_size, self.scale, self.num_kv_heads = num_heads, head_size, scale, num_kv_heads
        self.layer_idx = layer_idx
        self.window = sliding_window or -1
        self.softcap = softcap
        self.sinks = sinks
        self.k_scale, self.v_scale = k_scale, v_scale

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: Optional[torch.Tensor] = None,
                rope=None) -> torch.Tensor:
        """``q [T, Hq*D]``, ``k, v [T, Hkv*D]`` (views into the qkv GEMM output are fine).
        With ``rope`` given, RoPE is applied inside the cache-write kernel."""
        ctx = get_forward_context()
        md = ctx.attn_metadata
        kv_cache, kv_scales = ctx.kv_caches[self.layer_idx]
        T = q.shape[0]
        if isinstance(kv_scales, tq.TqFormat):
            return self._forward_turboquant(q, k, v, positions, rope, md, kv_cache, kv_scales)
        if "dcp_ctx_lens" in md.extra:
            return self._forward_dcp(q, k, v, positions, rope, md, kv_cache, kv_scales)
        pcp_slots = md.extra.get("pcp_slots_all")
        if pcp_slots is not None:
            # prefill context parallel: this copy computed a slice of every chunk; the copies exchange their K / V
            # rows and each writes all of them into its own (replicated) cache - parallel/pcp.py
            from ..parallel import state as ps

            if rope is not None:
                ops.rotary_embedding(positions, q, k, self.head_size, rope.cos_sin_cache, rope.is_neox)
            g, sizes = ps.get_pcp_group(), md.extra["pcp_sizes"]
            k_all, v_all = g.all_gatherv(k.contiguous(), sizes), g.all_gatherv(v.contiguous(), sizes)
            ops.reshape_and_cache(k_all, v_all, kv_cache, pcp_slots, kv_scales, self.k_scale, self.v_scale)
        elif rope is not None:
            ops.rope_and_cache(positions, q, k, v, self.head_size, rope.cos_sin_cache, rope.is_neox, kv_cache,
                               md.slot_mapping, kv_scales, self.k_scale, self.v_scale)
        else:
            ops.reshape_and_cache(k, v, kv_cache, md.slot_mapping, kv_scales, self.k_scale, self.v_scale)
        q3 = q.reshape(T, self.num_heads, self.head_size)
        if not q3.is_contiguous() and q3.stride(1) != self.head_size:
            q3 = q3.contiguous()
        out = torch.empty(T, self.num_heads, self.head_size, dtype=q.dtype, device=q.device)
        nd, ndt = md.num_decodes, md.num_decode_tokens
        if "cascade_blocks" in md.extra and self.window == -1 and self.alibi_slopes is None and self.sinks is None:
            return self._forward_cascade(q3, out, md, kv_cache, kv_scales)
        if nd > 0:
            ops.paged_attention_decode(q3[:ndt], kv_cache, md.block_table[:nd], md.seq_lens[:nd], self.scale,
                                       out=out[:ndt], kv_scales=kv_scales, window=self.window, softcap=self.softcap,
                                       sinks=self.sinks, num_splits=md.decode_num_splits, max_seq_len=md.max_seq_len,
                                       k_scale=self.k_scale, v_scale=self.v_scale, workspace=md.decode_workspace,
                                       alibi_slopes=self.alibi_slopes)
        if md.num_prefills > 0:
            ops.paged_attention_prefill(q3[ndt:], kv_cache, md.block_table[nd:], md.seq_lens[nd:],
                                        md.prefill_query_start_loc, self.scale, out=out[ndt:], kv_scales=kv_scales,
                                        max_q_len=md.max_prefill_query_len, window=self.window, softcap=self.softcap,
                                        sinks=self.sinks, k_scale=self.k_scale, v_scale=self.v_scale,
                                        max_seq_len=md.max_seq_len, alibi_slopes=self.alibi_slopes)
        return out.reshape(T, self.num_heads * self.head_size)

    def _forward_cascade(self, q3, out, md, kv_cache, kv_scales) -> torch.Tensor:
        """Shared-prefix (cascade) attention: the leading ``cascade_blocks`` cache blocks are the same physical blocks
        for every request of the step, so all of the step's query tokens attend them in ONE pass (one pseudo request,
        no causal mask: the prefix precedes every query), every request attends the rest of its own context, and the
        two partial results are merged by their log-sum-exps.  The prefix is read once per step instead of once per
        request.  Mirrors the cascade path of vllm_metax/v1/attention/backends/flash_attn.py (``use_cascade_attention``
        / ``cascade_attention``: prefix pass + suffix pass + ``merge_attn_states``)."""
        T, H, D = q3.shape
        dev = q3.device
        n = md.extra["cascade_blocks"]
        nd, ndt = md.num_decodes, md.num_decode_tokens
        common = dict(kv_scales=kv_scales, softcap=self.softcap, k_scale=self.k_scale, v_scale=self.v_scale)
        o_p = torch.empty(T, H, D, dtype=q3.dtype, device=dev)
        lse_p = torch.empty(H, T, dtype=torch.float32, device=dev)
        ops.paged_attention_prefill(q3, kv_cache, md.block_table[:1, :n].contiguous(), md.extra["cascade_seq_len"],
                                    md.extra["cascade_qsl"], self.scale, out=o_p, lse_out=lse_p, max_q_len=T,
                                    causal=False, max_seq_len=n * md.block_size, **common)
        table, lens = md.extra["cascade_suffix_table"], md.extra["cascade_suffix_lens"]
        o_s = torch.empty(T, H, D, dtype=q3.dtype, device=dev)
        parts = []
        if nd > 0:
            lse_d = torch.empty(H, ndt, dtype=torch.float32, device=dev)
            ops.paged_attention_decode(q3[:ndt], kv_cache, table[:nd], lens[:nd], self.scale, out=o_s[:ndt],
                                       lse_out=lse_d, max_seq_len=md.max_seq_len, **common)
            parts.append(lse_d)
        if md.num_prefills > 0:
            lse_f = torch.empty(H, T - ndt, dtype=torch.float32, device=dev)
            ops.paged_attention_prefill(q3[ndt:], kv_cache, table[nd:], lens[nd:], md.prefill_query_start_loc, self.scale,
                                        out=o_s[ndt:], lse_out=lse_f, max_q_len=md.max_prefill_query_len,
                                        max_seq_len=md.max_seq_len, **common)
            parts.append(lse_f)
        lse_s = parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)
        out = ops.merge_attn_states(o_p, lse_p, o_s, lse_s.contiguous())
        return out.reshape(T, H * D)

    def _forward_dcp(self, q, k, v, positions, rope, md, kv_cache, kv_scales) -> torch.Tensor:
        """Decode context parallel: this rank's cache holds every dcp-th token of each sequence (the slot mapping is
        -1 for the others).  Decode rows: all-gather q over the group's heads, attend the local shard, combine the
        partial outputs by their log-sum-exp and keep this rank's heads.  Prefill rows: causal attention over the
        chunk's own fresh K / V (every rank has them - its KV heads are replicated over the group) merged with the
        same gather / local / combine pass over the cached context, which needs no mask because all of it precedes
        the chunk.  Mirrors vllm_metax/v1/attention/backends/flash_attn.py:1450-1610."""
        from ..parallel import dcp
        from ..parallel import state as ps

        g = ps.get_dcp_group()
        d = g.world_size
        T, H, D = q.shape[0], self.num_heads, self.head_size
        if rope is not None:
            ops.rope_and_cache(positions, q, k, v, D, rope.cos_sin_cache, rope.is_neox, kv_cache, md.slot_mapping,
                               kv_scales, self.k_scale, self.v_scale)
        else:
            ops.reshape_and_cache(k, v, kv_cache, md.slot_mapping, kv_scales, self.k_scale, self.v_scale)
        q3 = q.reshape(T, H, D)
        out = torch.empty(T, H, D, dtype=q.dtype, device=q.device)
        nd, ndt = md.num_decodes, md.num_decode_tokens
        common = dict(kv_scales=kv_scales, window=self.window, softcap=self.softcap, k_scale=self.k_scale,
                      v_scale=self.v_scale, alibi_slopes=None)
        assert self.alibi_slopes is None and self.sinks is None, "ALiBi / sinks are not combined with DCP"

        def masked(o, lse, empty_rows):           # rows whose local shard is empty contribute nothing
            lse = torch.where(empty_rows[None, :], torch.full_like(lse, float("-inf")), lse)
            return torch.where(empty_rows[:, None, None], torch.zeros_like(o), o), lse.t().contiguous()

        if nd > 0:
            lens = md.seq_lens[:nd]

            def attend_decode(q_all):
                o = torch.empty(ndt, H * d, D, dtype=q.dtype, device=q.device)
                lse = torch.empty(H * d, ndt, dtype=torch.float32, device=q.device)
                ops.paged_attention_decode(q_all, kv_cache, md.block_table[:nd], lens.clamp_min(1), self.scale, out=o,
                                           lse_out=lse, num_splits=md.decode_num_splits, max_seq_len=md.max_seq_len,
                                           workspace=md.decode_workspace, **common)
                return masked(o, lse, lens == 0)

            out[:ndt] = dcp.decode_attention(q3[:ndt].contiguous(), attend_decode, g)
        if md.num_prefills > 0:
            Tp = T - ndt
            cu = md.prefill_query_start_loc
            Hkv = self.num_kv_heads
            qp = q3[ndt:].contiguous()
            kp = k[ndt:].reshape(Tp, Hkv, D).contiguous()
            vp = v[ndt:].reshape(Tp, Hkv, D).contiguous()
            o_self = torch.empty(Tp, H, D, dtype=q.dtype, device=q.device)
            lse_self = torch.empty(H, Tp, dtype=torch.float32, device=q.device)
            ops.varlen_attention(qp, kp, vp, cu, cu, self.scale, out=o_self, max_q_len=md.max_prefill_query_len,
                                 causal=True, window=self.window, softcap=self.softcap, lse_out=lse_self)
            if md.extra["dcp_any_context"]:
                ctx = md.extra["dcp_ctx_lens"][nd:]
                qlens = (cu[1:] - cu[:-1]).long()
                empty_tok = torch.repeat_interleave(ctx == 0, qlens, output_size=Tp)

                def attend_context(q_all):
                    o = torch.empty(Tp, H * d, D, dtype=q.dtype, device=q.device)
                    lse = torch.empty(H * d, Tp, dtype=torch.float32, device=q.device)
                    ops.paged_attention_prefill(q_all, kv_cache, md.block_table[nd:], ctx.clamp_min(1), cu, self.scale,
                                                out=o, lse_out=lse, max_q_len=md.max_prefill_query_len, causal=False,
                                                max_seq_len=md.max_seq_len, **{k_: v_ for k_, v_ in common.items()
                                                                               if k_ != "window"})
                    return masked(o, lse, empty_tok)

                o_ctx, lse_ctx = dcp.decode_attention(qp, attend_context, g, return_lse=True)
                out[ndt:] = ops.merge_attn_states(o_ctx, lse_ctx.t().contiguous(), o_self, lse_self)
            else:
                out[ndt:] = o_self
        return out.reshape(T, H * D)

    def _forward_turboquant(self, q, k, v, positions, rope, md, cache, fmt) -> torch.Tensor:
        """TurboQuant cache: RoPE, quantising store, then decode rows straight from the compressed slots and prefill
        rows against the de-quantised context (the cache is the only source of K / V, so a chunk sees its own keys
        through the same quantiser as every later step will).  Mirrors the split of
        vllm_metax/v1/attention/backends/turboquant_attn.py:286-942."""
        T = q.shape[0]
        if rope is not None:
            ops.rotary_embedding(positions, q, k, self.head_size, rope.cos_sin_cache, rope.is_neox)
        tq.store(k, v, cache, md.slot_mapping[:T], fmt)
        q3 = q.reshape(T, self.num_heads, self.head_size)
        if not q3.is_contiguous():
            q3 = q3.contiguous()
        out = torch.empty(T, self.num_heads, self.head_size, dtype=q.dtype, device=q.device)
        nd, ndt = md.num_decodes, md.num_decode_tokens
        if nd > 0 and ndt == nd:
            tq.decode_attention(q3[:nd], cache, md.block_table[:nd], md.seq_lens[:nd], self.scale, fmt, out=out[:nd])
            first = nd
        else:
            first = 0                   # multi-token decode rows (speculative drafts) take the prefill route
        if first < md.num_reqs:
            bs = cache.shape[1]
            lens = md.seq_lens[first: md.num_reqs].cpu()
            qsl = md.query_start_loc[first: md.num_reqs + 1]
            t0 = 0 if first == 0 else ndt
            slots = torch.cat([tq._slots_of(md.block_table[first + i], int(L), bs) for i, L in enumerate(lens.tolist())])
            kd, vd = tq.dequant(cache, slots, fmt, q.dtype)
            cu_k = torch.zeros(lens.numel() + 1, dtype=torch.int32)
            cu_k[1:] = lens.cumsum(0)
            cu_q = (qsl - qsl[0]).int()
            ops.varlen_attention(q3[t0:], kd, vd, cu_q, cu_k.to(q.device), self.scale, out=out[t0:],
                                 max_q_len=md.max_query_len, causal=True, window=self.window, softcap=self.softcap,
                                 sinks=self.sinks)
        return out.reshape(T, self.num_heads * self.head_size)
