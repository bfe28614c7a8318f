"""Per-step attention metadata and the forward context that carries it to the layers.

The flat token buffer of a step is ordered decode-first: tokens ``[0, num_decode_tokens)``
belong to ``num_decodes`` sequences with one query token each, the rest to
prefill / chunked-prefill sequences.  All index tensors live on the device of the
model; the ``*_cpu`` copies avoid device syncs in host code.

Parity: the fields mirror upstream CommonAttentionMetadata (query_start_loc, seq_lens,
block_table_tensor, slot_mapping, max_query_len, max_seq_len) that every reference
backend builds its metadata from (vllm_metax/v1/attention/backends/flash_attn.py:246-325).
"""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class AttentionMetadata:
    num_tokens: int
    num_reqs: int
    num_decodes: int                 # leading requests with exactly one query token (and past context)
    num_decode_tokens: int
    query_start_loc: torch.Tensor    # int32 [num_reqs+1]
    seq_lens: torch.Tensor           # int32 [num_reqs]  (context + new tokens)
    block_table: torch.Tensor        # int32 [num_reqs, max_blocks]
    slot_mapping: torch.Tensor       # int64 [num_tokens]
    max_query_len: int
    max_seq_len: int
    block_size: int
    query_start_loc_cpu: Optional[torch.Tensor] = None
    seq_lens_cpu: Optional[torch.Tensor] = None
    # prefill slice views (rebased so that the first prefill token is 0)
    prefill_query_start_loc: Optional[torch.Tensor] = None
    max_prefill_query_len: int = 0
    decode_num_splits: int = 0       # 0 = choose from shapes; fixed under CUDA graphs
    decode_workspace: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)

    @property
    def num_prefills(self) -> int:
        return self.num_reqs - self.num_decodes

    @property
    def num_prefill_tokens(self) -> int:
        return self.num_tokens - self.num_decode_tokens


@dataclass
class ForwardContext:
    attn_metadata: Optional[AttentionMetadata]
    kv_caches: list = field(default_factory=list)    # per layer: tensor or tuple of tensors
    positions: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)


class _Local(threading.local):
    ctx: Optional[ForwardContext] = None


_LOCAL = _Local()        # per thread: engines of one process that step on different threads do not see each other's step


def get_forward_context() -> ForwardContext:
    ctx = _LOCAL.ctx
    assert ctx is not None, "forward context not set"
    return ctx


@contextlib.contextmanager
def set_forward_context(ctx: ForwardContext):
    prev = _LOCAL.ctx
    _LOCAL.ctx = ctx
    try:
        yield
    finally:
        _LOCAL.ctx = prev


def merge_multimodal_embeddings(h: torch.Tensor) -> torch.Tensor:
    """Overwrite the rows of image / audio placeholder tokens with the encoder's projected features (called by the text
    decoders right after their embedding lookup; a no-op for text-only steps).  The runner lists the rows of this
    step's chunk in ``extra["mm_rows"]`` and their features, in the same order, in ``extra["mm_embeds"]``."""
    ctx = _LOCAL.ctx
    md = ctx.attn_metadata if ctx is not None else None
    if md is None or "mm_embeds" not in md.extra:
        return h
    emb = md.extra["mm_embeds"]
    H = h.shape[1]
    if emb.shape[1] > H:          # DeepStack models: the wider rows carry extra feature levels for the first layers
        md.extra["mm_deepstack"] = emb[:, H:].reshape(emb.shape[0], -1, H)
        emb = emb[:, :H]
    return h.index_copy_(0, md.extra["mm_rows"], emb.to(h.dtype))
