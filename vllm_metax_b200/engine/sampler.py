"""Batch sampling driver: penalties -> temperature / top-k / top-p / min-p -> token.

Randomness is one uniform number per request per step drawn on the host from the request's own
generator (seeded requests are reproducible regardless of batch composition); the device kernel
turns it into a token by inverse CDF over the filtered distribution.
"""
from __future__ import annotations

import random

import torch

from .. import _custom_ops as ops

_global_rng = random.Random(0)


def seed_global(seed: int) -> None:
    global _global_rng
    _global_rng = random.Random(seed)


def _uniform_for(req) -> float:
    """A seeded request draws from its own stream, kept on the request (two engines in one process, or a reused
    request id, never share one)."""
    if req.params.seed is None:
        return _global_rng.random()
    rng = getattr(req, "_sample_rng", None)
    if rng is None:
        rng = req._sample_rng = random.Random(req.params.seed)
    return rng.random()


def forget(request_id: str) -> None:
    """Kept for callers of earlier versions: the streams live on the requests and need no clean-up."""


def sample_batch(logits: torch.Tensor, reqs, out: torch.Tensor) -> torch.Tensor:
    dev = logits.device
    B, V = logits.shape
    if any(r.params.constrained for r in reqs):
        from .structured import apply_constraints

        logits = apply_constraints(logits, reqs)
    if any(r.params.needs_penalties for r in reqs):
        logits = logits.float() if logits.dtype != torch.float32 else logits.clone()
        counts = torch.zeros(B, V, dtype=torch.int32)
        pmask = torch.zeros(B, V, dtype=torch.int32)
        for i, r in enumerate(reqs):
            if r.output_token_ids:
                idx = torch.tensor(r.output_token_ids)
                counts[i].index_add_(0, idx, torch.ones_like(idx, dtype=torch.int32))
            pmask[i, torch.tensor(r.prompt_token_ids)] = 1
        rep = torch.tensor([r.params.repetition_penalty for r in reqs], dtype=torch.float32, device=dev)
        pres = torch.tensor([r.params.presence_penalty for r in reqs], dtype=torch.float32, device=dev)
        freq = torch.tensor([r.params.frequency_penalty for r in reqs], dtype=torch.float32, device=dev)
        ops.apply_penalties(logits, pmask.to(dev), counts.to(dev), rep, pres, freq)
    temp = torch.tensor([r.params.temperature for r in reqs], dtype=torch.float32, device=dev)
    top_k = torch.tensor([r.params.top_k for r in reqs], dtype=torch.int32, device=dev)
    top_p = torch.tensor([r.params.top_p for r in reqs], dtype=torch.float32, device=dev)
    min_p = torch.tensor([r.params.min_p for r in reqs], dtype=torch.float32, device=dev)
    uni = torch.tensor([_uniform_for(r) for r in reqs], dtype=torch.float32, device=dev)
    return ops.sample(logits, temp, top_k, top_p, min_p, uni, out)
