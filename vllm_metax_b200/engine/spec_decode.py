"""Speculative decoding: draft proposers and the verification rule.

A proposer attaches ``spec_token_ids`` to a running request; the scheduler then feeds
``[last token, draft_1 .. draft_k]`` in one step, the model runner samples the target token of every fed
position, and ``Scheduler.update`` keeps drafts while they equal the target token (``verify`` below states
the rule).  For deterministic drafts this is exact rejection sampling: a token sampled from the target
distribution p equals the draft with probability p(draft), and conditioned on a mismatch it is distributed as
the residual ``p restricted to != draft`` - the same output distribution as decoding without drafts, and
bit-identical tokens under greedy sampling.

* ``NgramProposer``   prompt-lookup decoding: the longest recent n-gram that occurred earlier in the sequence
                      proposes the tokens that followed it.
* ``MTPProposer``     multi-token-prediction heads (``models/deepseek_mtp.py``): one extra decoder layer per
                      look-ahead step fed with the target model's hidden states.

Parity: the reference serves MTP / EAGLE / n-gram speculative decoding through vLLM's v1 spec-decode runner
(models/deepseek_mtp.py, models/step3p5_mtp.py, patch/performance/speculative_decode_perf.py:29-155 for the
query-length bucketing of multi-token decodes).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class SpeculativeConfig:
    method: str = "ngram"                  # "ngram" | "mtp" | "eagle"
    num_speculative_tokens: int = 4
    prompt_lookup_max: int = 4
    prompt_lookup_min: int = 1
    model: object = None                   # eagle: draft checkpoint directory, config dict or ModelConfig
    own_embeddings: bool = False           # eagle: keep the draft's own embedding / head instead of the target's

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["SpeculativeConfig"]:
        if not d:
            return None
        known = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        return cls(**known)


def verify(drafts: Sequence[int], targets: Sequence[int]) -> list[int]:
    """Tokens produced by one verified step: the accepted draft prefix plus the first target token after it.
    ``targets`` has ``len(drafts) + 1`` entries (one per fed position)."""
    acc = 0
    while acc < len(drafts) and drafts[acc] == targets[acc]:
        acc += 1
    return list(targets[: acc + 1])


class NgramProposer:
    def __init__(self, cfg: SpeculativeConfig):
        self.k = cfg.num_speculative_tokens
        self.max_n, self.min_n = cfg.prompt_lookup_max, max(1, cfg.prompt_lookup_min)

    def propose(self, token_ids: Sequence[int]) -> list[int]:
        L = len(token_ids)
        for n in range(min(self.max_n, L - 1), self.min_n - 1, -1):
            tail = list(token_ids[L - n:])
            # most recent earlier occurrence of the tail
            for start in range(L - n - 1, -1, -1):
                if list(token_ids[start:start + n]) == tail:
                    follow = list(token_ids[start + n: start + n + self.k])
                    if follow:
                        return follow
        return []


def make_proposer(cfg: Optional[SpeculativeConfig], engine=None):
    if cfg is None:
        return None
    if cfg.method == "ngram":
        return NgramProposer(cfg)
    if cfg.method == "mtp":
        from ..models.deepseek_mtp import MTPProposer

        return MTPProposer(cfg, engine)
    if cfg.method == "eagle":
        import copy

        from ..models.deepseek_mtp import MTPProposer

        if cfg.model is None:                                   # a one-layer head with the target's dimensions
            draft = copy.copy(engine.cfg.model)
            draft.num_hidden_layers = 1
        else:
            from .llm import _resolve_model

            draft, _ = _resolve_model(cfg.model, dtype=engine.cfg.model.dtype)
        return MTPProposer(cfg, engine, architecture="EagleLlamaForCausalLM", draft_model=draft)
    raise ValueError(f"unknown speculative method {cfg.method!r}")
