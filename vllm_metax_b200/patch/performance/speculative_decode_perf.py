"""Batch order for speculative decoding: decodes first, SORTED BY QUERY LENGTH, then chunked-prefill
extends, then first-chunk prefills.

With multi-token (MTP / EAGLE / n-gram) decoding the requests of one step carry 1..k+1 query tokens.
The decode attention kernel is launched per query-length bucket, so requests of equal length must be
contiguous; upstream only splits decode / prefill.  ``plan_order`` computes the stable target order,
``swaps_for`` turns it into the minimal list of pairwise swaps (cycle decomposition) that
``InputBatch.swap_states`` applies.
Parity: vllm_metax/patch/performance/speculative_decode_perf.py:29-155.
"""
from __future__ import annotations

import numpy as np

from .. import utils


def plan_order(num_scheduled: np.ndarray, num_computed: np.ndarray, num_prompt: np.ndarray,
               decode_threshold: int) -> tuple[np.ndarray, dict[str, int]]:
    """Permutation ``order`` (new position -> old index) and region sizes."""
    n = len(num_scheduled)
    has_ctx = num_computed > 0
    below = num_scheduled <= decode_threshold
    done = num_computed >= num_prompt
    region = np.full(n, 3, dtype=np.int64)                 # 3: prefill (no context yet)
    region[has_ctx & ~below] = 2                           # 2: long extend
    region[has_ctx & below & ~done] = 1                    # 1: short extend
    region[has_ctx & below & done] = 0                     # 0: decode
    qlen_key = np.where(region == 0, num_scheduled, 0)     # only decodes are sorted by length
    order = np.lexsort((np.arange(n), qlen_key, region))   # stable: region, then qlen, then old index
    sizes = {"decode": int((region == 0).sum()), "short_extend": int((region == 1).sum()),
             "long_extend": int((region == 2).sum()), "prefill": int((region == 3).sum())}
    return order, sizes


def swaps_for(order: np.ndarray) -> list[tuple[int, int]]:
    """Pairwise swaps that turn the identity arrangement into ``order``."""
    cur = list(range(len(order)))          # cur[pos] = old index now sitting at pos
    where = list(range(len(order)))        # where[old] = pos
    out: list[tuple[int, int]] = []
    for pos, want in enumerate(order.tolist()):
        if cur[pos] == want:
            continue
        src = where[want]
        out.append((pos, src))
        a, b = cur[pos], cur[src]
        cur[pos], cur[src] = b, a
        where[a], where[b] = src, pos
    return out


def reorder_batch(input_batch, scheduler_output, decode_threshold: int) -> bool:
    n = len(input_batch.req_ids)
    sched = np.array([scheduler_output.num_scheduled_tokens[r] for r in input_batch.req_ids], dtype=np.int64)
    order, _ = plan_order(sched, np.asarray(input_batch.num_computed_tokens_cpu[:n]),
                          np.asarray(input_batch.num_prompt_tokens[:n]), decode_threshold)
    swaps = swaps_for(order)
    for i, j in swaps:
        input_batch.swap_states(i, j)
    return bool(swaps)


def _may_reorder_batch(self, scheduler_output) -> None:
    if len(self.kv_cache_config.kv_cache_groups) == 0:
        return
    if self.reorder_batch_threshold is not None:
        reorder_batch(self.input_batch, scheduler_output, self.reorder_batch_threshold)


try:
    import vllm.v1.worker.gpu_model_runner  # noqa: F401

    utils.apply_patch("vllm.v1.worker.gpu_model_runner", "GPUModelRunner._may_reorder_batch", _may_reorder_batch)
except ImportError:
    pass
