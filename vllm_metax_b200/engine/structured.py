"""Constrained decoding: the sampler masks the logits of a request down to the tokens its constraint allows.

* ``allowed_token_ids`` - a fixed allow-list for every step.
* ``logit_bias`` - additive per-token biases.
* ``guided_choice`` - the output must be exactly one of the given alternatives (token-id lists, or strings when a
  tokenizer is attached).  The alternatives form a token trie; the allowed set of a step is the children of the node
  reached by the tokens generated so far, so the state is a pure function of the request's output and survives
  preemption and recomputation without bookkeeping.  The request stops as soon as it has produced a complete
  alternative.

Regular-expression and JSON-schema guidance need a character-level automaton intersected with the vocabulary; they
are not built (``guided_regex`` / ``guided_json`` raise).  Parity: the structured-outputs examples of the reference
(examples/features/structured_outputs in its tree) run on upstream's backends.
"""
from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch


class TokenTrie:
    def __init__(self, alternatives: Iterable[Sequence[int]]):
        self.root: dict = {}
        n = 0
        for alt in alternatives:
            alt = list(alt)
            if not alt:
                raise ValueError("an empty alternative cannot be generated")
            node = self.root
            for t in alt:
                node = node.setdefault(int(t), {})
            node[None] = True            # end marker
            n += 1
        if n == 0:
            raise ValueError("guided_choice needs at least one alternative")

    def _walk(self, prefix: Sequence[int]) -> Optional[dict]:
        node = self.root
        for t in prefix:
            node = node.get(int(t))
            if node is None:
                return None
        return node

    def allowed_after(self, prefix: Sequence[int]) -> list[int]:
        """Tokens that keep ``prefix`` a prefix of some alternative ([] when it is complete or off the trie)."""
        node = self._walk(prefix)
        return [] if node is None else [t for t in node if t is not None]

    def complete(self, prefix: Sequence[int]) -> bool:
        """True when ``prefix`` is an alternative and no longer one extends it - or when it left the trie."""
        node = self._walk(prefix)
        return node is None or (None in node and len(node) == 1)


def resolve_choices(choices, tokenizer) -> list[list[int]]:
    out = []
    for c in choices:
        if isinstance(c, str):
            if tokenizer is None:
                raise ValueError("string alternatives need a tokenizer; pass token-id lists instead")
            out.append(list(tokenizer.encode(c, add_special_tokens=False)))
        else:
            out.append([int(t) for t in c])
    return out


def constraint_of(req) -> Optional[list[int]]:
    """Allowed token ids for the request's next step, or None when it is unconstrained."""
    p = req.params
    allowed: Optional[set] = None
    trie = getattr(p, "_trie", None)
    if trie is not None:
        nxt = trie.allowed_after(req.output_token_ids)
        if not nxt and req.eos_token_id is not None:
            nxt = [req.eos_token_id]
        allowed = set(nxt)
    if p.allowed_token_ids:
        a = set(p.allowed_token_ids)
        allowed = a if allowed is None else (allowed & a)
    return None if allowed is None else sorted(allowed)


def apply_constraints(logits: torch.Tensor, reqs) -> torch.Tensor:
    """Returns logits (a float32 copy when anything is changed) with biases added and disallowed tokens at -inf."""
    touched = False
    for i, r in enumerate(reqs):
        p = r.params
        allowed = constraint_of(r)
        if allowed is None and not p.logit_bias:
            continue
        if not touched:
            logits = logits.float().clone()
            touched = True
        if p.logit_bias:
            idx = torch.tensor(list(p.logit_bias.keys()), dtype=torch.long, device=logits.device)
            val = torch.tensor(list(p.logit_bias.values()), dtype=torch.float32, device=logits.device)
            logits[i].index_add_(0, idx, val)
        if allowed is not None:
            keep = torch.tensor(allowed, dtype=torch.long, device=logits.device)
            row = torch.full_like(logits[i], float("-inf"))
            row[keep] = logits[i][keep]
            logits[i] = row
    return logits
