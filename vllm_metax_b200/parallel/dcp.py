"""Decode context parallelism (DCP): the KV cache of a sequence is sharded along the sequence, interleaved over
the ranks of the DCP group (token ``i`` lives on rank ``i % dcp``), so a long context costs every rank 1/dcp of
the cache memory and of the decode read traffic.

A decode step then is:
  1. all-gather the query over the head dimension (the DCP group is a sub-group of the TP group, every rank owns
     different heads) - ``gather_query``;
  2. every rank attends ALL heads against its local KV shard and returns the partial output with its
     log-sum-exp;
  3. ``combine_partials``: all-gather the LSEs, rescale each partial by ``exp(lse_r - lse_total)`` and
     reduce-scatter the outputs over heads, which leaves every rank with the exact attention output of its heads.

The helpers below also give the local view of a sequence (``local_seq_lens``, ``owns_position``) that the cache
writer and the metadata builder need.  Tensors on CPU ranks go through Gloo, which is how the protocol is tested.

Parity: vllm_metax/v1/attention/backends/flash_attn.py:1450-1610 (all-gather q, context attention over the local
shard, ``cp_lse_ag_out_rs``), vllm_metax/v1/attention/backends/mla/mla_attention.py:858-899 (MLA decode).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from .state import Group


def local_seq_lens(seq_lens: torch.Tensor, dcp: int, rank: int) -> torch.Tensor:
    """Tokens of each sequence that rank ``rank`` holds under the interleaved layout."""
    return (seq_lens - rank + dcp - 1).clamp_min(0) // dcp


def owns_position(positions: torch.Tensor, dcp: int, rank: int) -> torch.Tensor:
    """Mask of the new tokens whose K/V this rank stores (the others write nothing: slot -1)."""
    return positions % dcp == rank


def local_slot_mapping(slot_mapping: torch.Tensor, positions: torch.Tensor, dcp: int, rank: int) -> torch.Tensor:
    """Slot mapping of this rank: tokens owned elsewhere get -1, which every cache-write kernel skips."""
    return torch.where(owns_position(positions, dcp, rank), slot_mapping, torch.full_like(slot_mapping, -1))


def gather_query(q: torch.Tensor, group: Group) -> torch.Tensor:
    """``[T, H_local, D]`` -> ``[T, H_local * dcp, D]`` in rank order."""
    return q if group.world_size == 1 else group.all_gather(q.contiguous(), 1)


def combine_partials(out: torch.Tensor, lse: torch.Tensor, group: Group, return_lse: bool = False):
    """``out [T, H_all, Dv]`` and ``lse [T, H_all]`` (natural log, ``-inf`` where the local shard was empty) computed
    against the local KV shard -> exact output of this rank's heads ``[T, H_all / dcp, Dv]`` (+ their total LSE)."""
    n = group.world_size
    if n == 1:
        return (out, lse) if return_lse else out
    T, H, Dv = out.shape
    assert H % n == 0
    lses = group.all_gather(lse.float().contiguous().unsqueeze(0), 0)          # [dcp, T, H]
    total = torch.logsumexp(lses, dim=0)                                       # [T, H]
    w = torch.exp(lse.float() - total)
    w = torch.where(torch.isfinite(w), w, torch.zeros_like(w))                 # empty shard (or empty everywhere)
    scaled = (out.float() * w.unsqueeze(-1)).to(out.dtype if out.dtype != torch.float32 else torch.float32)
    mine = group.reduce_scatter(scaled, 1)                                     # heads of this rank
    if not return_lse:
        return mine
    hl = H // n
    r = group.rank_in_group
    return mine, total[:, r * hl:(r + 1) * hl].contiguous()


def decode_attention(q_local: torch.Tensor, attend_local: Callable[[torch.Tensor], Tuple[torch.Tensor, torch.Tensor]],
                     group: Group, return_lse: bool = False):
    """One DCP decode: ``attend_local(q_all) -> (out [T, H_all, Dv], lse [T, H_all])`` runs this package's decode
    kernel (``paged_attention_decode`` / ``mla_decode`` with ``lse_out``) on the rank's shard of the cache."""
    q_all = gather_query(q_local, group)
    out, lse = attend_local(q_all)
    return combine_partials(out, lse, group, return_lse)


def shard_kv_interleaved(k: torch.Tensor, dcp: int, rank: int, start: int = 0) -> torch.Tensor:
    """Rows of ``k [L, ...]`` (positions ``start .. start + L - 1``) that live on ``rank``."""
    first = (rank - start) % dcp
    return k[first::dcp]
