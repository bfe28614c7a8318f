"""Attention backends in vLLM's v1 interface (``AttentionBackend`` / ``AttentionMetadataBuilder`` /
``AttentionImpl``) over this package's kernels.  Used when the package runs as a vLLM platform plugin;
the standalone engine uses ``layers/attention.py`` and ``layers/mla.py`` directly.

* ``PagedGQABackend``    dense GQA/MQA/MHA: KV cache ``[blocks, 2, block_size, kv_heads, head]``, decode by
                          the split-KV kernel, prefill / chunked prefill by the tcgen05 kernel.
* ``MLABackend``          absorbed MLA decode over the 576-wide latent cache (bf16 or fp8_ds_mla records).
* ``MLASparseBackend``    the same kernel with per-token top-k indices (DeepSeek-V3.2).

The builders split each batch decode-first exactly like the standalone model runner (requests with one
scheduled token and computed context come first; the platform sets the reorder threshold).

Parity: vllm_metax/v1/attention/backends/flash_attn.py:246-435 (metadata builder, per-query-length decode
buckets), flashinfer.py, triton_attn.py, mla/flashmla.py, mla/flashmla_sparse.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

from . import _custom_ops as ops

try:
    from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl,
                                           AttentionMetadataBuilder, AttentionType, CommonAttentionMetadata)

    _HAVE_VLLM = True
except Exception:  # pragma: no cover - standalone use without vLLM
    _HAVE_VLLM = False
    AttentionBackend = AttentionImpl = AttentionMetadataBuilder = object   # type: ignore
    CommonAttentionMetadata = object  # type: ignore

    class AttentionCGSupport:  # type: ignore
        UNIFORM_BATCH = 2
        NEVER = 0

    class AttentionType:  # type: ignore
        DECODER = "decoder"


@dataclass
class B200AttentionMetadata:
    num_actual_tokens: int
    num_decodes: int
    num_decode_tokens: int
    query_start_loc: torch.Tensor
    prefill_query_start_loc: Optional[torch.Tensor]
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    max_query_len: int
    max_prefill_query_len: int
    max_seq_len: int
    decode_query_len: int = 1
    topk_indices: Optional[torch.Tensor] = None


def split_decodes_and_prefills(query_start_loc_cpu: torch.Tensor, decode_threshold: int = 1) -> tuple[int, int]:
    """Leading requests whose query length is <= threshold are decodes: returns (num_decodes, num_decode_tokens)."""
    qlens = (query_start_loc_cpu[1:] - query_start_loc_cpu[:-1]).tolist()
    nd = 0
    for q in qlens:
        if q > decode_threshold:
            break
        nd += 1
    return nd, int(query_start_loc_cpu[nd])


class B200MetadataBuilder(AttentionMetadataBuilder):
    _cudagraph_support: ClassVar = AttentionCGSupport.UNIFORM_BATCH
    reorder_batch_threshold: int = 1

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        if _HAVE_VLLM:
            super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self.kv_cache_spec, self.device = kv_cache_spec, device

    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False) -> B200AttentionMetadata:
        m = common_attn_metadata
        nd, ndt = split_decodes_and_prefills(m.query_start_loc_cpu, self.reorder_batch_threshold)
        qsl = m.query_start_loc
        pre_qsl, max_pre = None, 0
        if nd < m.num_reqs:
            pre_qsl = (qsl[nd:] - qsl[nd]).to(torch.int32)
            pq = m.query_start_loc_cpu[nd + 1:] - m.query_start_loc_cpu[nd:-1]
            max_pre = int(pq.max())
        return B200AttentionMetadata(
            num_actual_tokens=m.num_actual_tokens, num_decodes=nd, num_decode_tokens=ndt,
            query_start_loc=qsl.to(torch.int32), prefill_query_start_loc=pre_qsl,
            seq_lens=m.seq_lens.to(torch.int32), block_table=m.block_table_tensor.to(torch.int32),
            slot_mapping=m.slot_mapping, max_query_len=m.max_query_len, max_prefill_query_len=max_pre,
            max_seq_len=m.max_seq_len)

    def build_for_cudagraph_capture(self, common_attn_metadata) -> B200AttentionMetadata:
        return self.build(0, common_attn_metadata)


class PagedGQAImpl(AttentionImpl):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes=None, sliding_window: Optional[int] = None, kv_cache_dtype: str = "auto",
                 logits_soft_cap: Optional[float] = None, attn_type: str = AttentionType.DECODER,
                 kv_sharing_target_layer_name: Optional[str] = None, sinks: Optional[torch.Tensor] = None, **_):
        if alibi_slopes is not None:
            raise NotImplementedError("ALiBi is handled by the varlen kernel, not by the paged backend")
        if attn_type != AttentionType.DECODER:
            raise NotImplementedError("only decoder self-attention uses the paged backend")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.window = sliding_window if isinstance(sliding_window, int) and sliding_window > 0 else -1
        self.softcap = float(logits_soft_cap or 0.0)
        self.kv_cache_dtype = kv_cache_dtype
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
        self.sinks = sinks

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not provided by this backend")
        T = query.shape[0]
        if output is None:
            output = torch.empty(T, self.num_heads * self.head_size, dtype=query.dtype, device=query.device)
        if attn_metadata is None:      # profiling run
            return output.fill_(0)
        md: B200AttentionMetadata = attn_metadata
        n = md.num_actual_tokens
        k_scale = float(getattr(layer, "_k_scale_float", 1.0))
        v_scale = float(getattr(layer, "_v_scale_float", 1.0))
        if self.kv_sharing_target_layer_name is None and key is not None:
            ops.reshape_and_cache(key[:n].reshape(n, -1), value[:n].reshape(n, -1), kv_cache, md.slot_mapping[:n], None,
                                  k_scale, v_scale)
        q3 = query[:n].reshape(n, self.num_heads, self.head_size)
        out3 = output[:n].view(n, self.num_heads, self.head_size)
        nd, ndt = md.num_decodes, md.num_decode_tokens
        if nd > 0:
            ops.paged_attention_decode(q3[:ndt], kv_cache, md.block_table[:nd], md.seq_lens[:nd], self.scale,
                                       out=out3[:ndt], window=self.window, softcap=self.softcap, sinks=self.sinks,
                                       max_seq_len=md.max_seq_len, k_scale=k_scale, v_scale=v_scale)
        if n > ndt:
            ops.paged_attention_prefill(q3[ndt:], kv_cache, md.block_table[nd:], md.seq_lens[nd:],
                                        md.prefill_query_start_loc, self.scale, out=out3[ndt:],
                                        max_q_len=md.max_prefill_query_len, window=self.window, softcap=self.softcap,
                                        sinks=self.sinks, k_scale=k_scale, v_scale=v_scale, max_seq_len=md.max_seq_len)
        return output


class PagedGQABackend(AttentionBackend):
    accept_output_buffer: bool = True
    supported_dtypes: ClassVar = [torch.bfloat16, torch.float16]
    supported_kv_cache_dtypes: ClassVar = ["auto", "bfloat16", "float16", "fp8", "fp8_e4m3", "int8"]

    @staticmethod
    def get_name() -> str:
        return "FLASH_ATTN"

    @staticmethod
    def get_impl_cls():
        return PagedGQAImpl

    @staticmethod
    def get_builder_cls():
        return B200MetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes():
        return [16, 32, 64, 128, 256]

    @classmethod
    def get_supported_head_sizes(cls) -> list[int]:
        return [64, 128, 256]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        return (num_blocks, 2, block_size, num_kv_heads, head_size)

    @classmethod
    def supports_sink(cls) -> bool:
        return True

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return tuple(capability)[0] == 10 if capability is not None else True


# ----------------------------------------------------------------------------- MLA
class MLAImpl:
    """Absorbed-MLA decode/prefill through ``ops.mla_decode``: queries already carry W_UK
    (``q [T, H, 576]`` = absorbed nope 512 + rope 64); output is the 512-wide latent, to be multiplied
    by W_UV by the caller."""

    def __init__(self, num_heads: int, scale: float, kv_cache_dtype: str = "auto", sparse: bool = False, **_):
        self.num_heads, self.scale, self.kv_cache_dtype, self.sparse = num_heads, float(scale), kv_cache_dtype, sparse

    def forward_mqa(self, q: torch.Tensor, kv_cache: torch.Tensor, md: B200AttentionMetadata) -> torch.Tensor:
        return ops.mla_decode(q, kv_cache, md.block_table, md.seq_lens, self.scale, query_start_loc=md.query_start_loc,
                              topk_indices=md.topk_indices if self.sparse else None, max_seq_len=md.max_seq_len)


class MLABackend(AttentionBackend):
    accept_output_buffer: bool = True

    @staticmethod
    def get_name() -> str:
        return "FLASHMLA"

    @staticmethod
    def get_impl_cls():
        return MLAImpl

    @staticmethod
    def get_builder_cls():
        return B200MetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes():
        return [64]

    @classmethod
    def get_supported_head_sizes(cls) -> list[int]:
        return [576]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if cache_dtype_str == "fp8_ds_mla":
            return (num_blocks, block_size, 656)
        return (num_blocks, block_size, head_size)

    @classmethod
    def is_mla(cls) -> bool:
        return True


class MLASparseBackend(MLABackend):
    @staticmethod
    def get_name() -> str:
        return "FLASHMLA_SPARSE"

    @classmethod
    def is_sparse(cls) -> bool:
        return True
