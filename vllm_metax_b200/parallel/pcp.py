"""Prefill context parallelism (PCP): ``pcp`` full copies of the (tensor-parallel) model split the tokens of every
prefill chunk between them, so the linear layers of a long prompt run on 1 / pcp of its tokens per copy.

Every copy runs the same scheduler.  For a scheduled request with ``n`` new tokens at positions ``p0 .. p0 + n - 1``

* ``n >= pcp`` (a prefill chunk): copy ``r`` takes the contiguous slice ``[a_r, b_r)`` - queries at ``a_r .. b_r - 1``
  attend keys ``< b_r``, which is a request of length ``b_r`` with ``b_r - a_r`` new tokens for the paged prefill
  kernel, so no kernel knows about the split;
* ``n < pcp`` (decode rows, tiny chunks): every copy computes the row itself.

After the K / V projection (and RoPE) the copies all-gather their rows and every copy writes ALL of them into its own
cache: the cache is replicated, so later chunks and the decode steps need no further exchange, and decode steps run
identically on all copies.  The request's last token of a chunk lives on the last copy, which samples and broadcasts
the tokens (``engine/model_runner.py``).

The reference takes PCP from upstream (``pcp_world_size`` in its attention metadata builders,
vllm_metax/v1/attention/backends/flash_attn.py:246-325 and mla_attention.py:2142-2297); this is the form with a replicated cache, for GQA caches (``layers/attention.py``) and for the MLA latent cache and
the sparse indexer's key cache (``layers/mla.py``).
"""
from __future__ import annotations

import numpy as np

from ..engine.scheduler import ScheduledRequest, SchedulerOutput


def slice_bounds(n: int, pcp: int, r: int) -> tuple[int, int]:
    """Offsets ``[a, b)`` inside a chunk of ``n >= pcp`` tokens that copy ``r`` computes (sizes differ by at most 1)."""
    base, extra = divmod(n, pcp)
    a = r * base + min(r, extra)
    return a, a + base + (1 if r < extra else 0)


def local_view(so: SchedulerOutput, pcp: int, r: int) -> SchedulerOutput:
    """The step as copy ``r`` runs it: sliced chunks (only the last copy samples them), whole small rows; decode rows
    first, as the runner expects."""
    rows = []
    for s in so.scheduled:
        if s.num_new_tokens >= pcp and pcp > 1:
            a, b = slice_bounds(s.num_new_tokens, pcp, r)
            rows.append(ScheduledRequest(s.request, b - a, s.start_pos + a, s.samples and r == pcp - 1, 0))
        else:
            rows.append(ScheduledRequest(s.request, s.num_new_tokens, s.start_pos, s.samples, s.num_spec))
    dec = [x for x in rows if x.is_decode]
    out = SchedulerOutput(scheduled=dec + [x for x in rows if not x.is_decode], num_decode=len(dec))
    out.preempted = so.preempted
    return out


def gathered_slots(so: SchedulerOutput, pcp: int, me: int, block_size: int) -> tuple[np.ndarray, list[int]]:
    """Cache slots of the all-gathered K / V rows (copy-major, each copy's rows in its ``local_view`` order) and the
    row count of every copy.  Rows that every copy computes itself are written from the local segment only (-1 in the
    segments of the other copies)."""
    sliced = {id(s.request): s.num_new_tokens >= pcp for s in so.scheduled}
    slots, sizes = [], []
    for r in range(pcp):
        n_rows = 0
        for s in local_view(so, pcp, r).scheduled:
            n = s.num_new_tokens
            n_rows += n
            if sliced[id(s.request)] or r == me:
                pos = np.arange(s.start_pos, s.start_pos + n)
                blk = np.asarray(s.request.block_ids, dtype=np.int64)
                slots.append(blk[pos // block_size] * block_size + pos % block_size)
            else:
                slots.append(np.full(n, -1, dtype=np.int64))
        sizes.append(n_rows)
    return (np.concatenate(slots) if slots else np.zeros(0, dtype=np.int64)), sizes


def sampling_requests(so: SchedulerOutput, pcp: int) -> list:
    """Requests whose tokens the last copy samples, in its row order (what every copy needs to read the broadcast)."""
    return [s.request for s in local_view(so, pcp, pcp - 1).scheduled if s.samples]
