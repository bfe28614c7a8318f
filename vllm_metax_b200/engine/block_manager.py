"""Paged KV-cache block pool with reference counting and optional prefix caching.

A block holds ``block_size`` consecutive token positions of one sequence.  With
prefix caching on, every *full* block is keyed by the hash of (parent hash,
its token ids); a new request walks its prompt and reuses matching blocks.
Freed blocks keep their hash until they are re-allocated (LRU order), so a
later request can still hit them.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

from .sampling_params import Request


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = False):
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_caching = enable_prefix_caching
        self.ref = [0] * num_blocks
        # free blocks in eviction order (oldest first); dict used as ordered set
        self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(num_blocks))
        self.hash_of: list[Optional[int]] = [None] * num_blocks
        self.block_of_hash: dict[int, int] = {}

    # ------------------------------------------------------------------ basic
    @property
    def num_free(self) -> int:
        return len(self.free)

    def _pop_free(self) -> int:
        bid, _ = self.free.popitem(last=False)
        h = self.hash_of[bid]
        if h is not None:
            if self.block_of_hash.get(h) == bid:
                del self.block_of_hash[h]
            self.hash_of[bid] = None
        return bid

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise RuntimeError("out of KV blocks")
        out = []
        for _ in range(n):
            bid = self._pop_free()
            self.ref[bid] = 1
            out.append(bid)
        return out

    def release(self, block_ids: list[int]) -> None:
        # free in reverse so that the tail of a sequence is evicted before its prefix
        for bid in reversed(block_ids):
            self.ref[bid] -= 1
            assert self.ref[bid] >= 0
            if self.ref[bid] == 0:
                self.free[bid] = None

    def reset_prefix_cache(self) -> None:
        """Forget every cached prefix (the weights changed: cached K/V no longer match).  Blocks in use keep their
        contents for their current owners but can no longer be hit by new requests."""
        self.block_of_hash.clear()
        self.hash_of = [None] * self.num_blocks

    # ------------------------------------------------------------------ prefix cache
    @staticmethod
    def chain_hash(parent: Optional[int], tokens: tuple) -> int:
        return hash((parent, tokens))

    def block_hashes(self, req: Request, upto_tokens: int) -> list[int]:
        """Hashes of the full blocks covering the first ``upto_tokens`` tokens (memoised on the request)."""
        bs = self.block_size
        nfull = upto_tokens // bs
        hs = req._hashes
        toks = None
        while len(hs) < nfull:
            if toks is None:
                toks = req.all_token_ids
            i = len(hs)
            root = None if req.lora_request is None else ("lora", req.lora_request.lora_int_id)   # K/V depend on the adapter
            if getattr(req, "mm_hash", None) is not None:                                         # ... and on the images
                root = (root, "mm", req.mm_hash)
            hs.append(self.chain_hash(hs[-1] if hs else root, tuple(toks[i * bs:(i + 1) * bs])))
        return hs[:nfull]

    def match_prefix(self, req: Request) -> list[int]:
        """Longest run of cached blocks for the request's tokens; takes a reference on each.

        At least one token is always left to compute so the request produces logits.
        """
        if not self.enable_prefix_caching:
            return []
        hashes = self.block_hashes(req, req.num_tokens - 1)
        out = []
        for h in hashes:
            bid = self.block_of_hash.get(h)
            if bid is None:
                break
            if self.ref[bid] == 0:
                self.free.pop(bid, None)
            self.ref[bid] += 1
            out.append(bid)
        return out

    def register_full_blocks(self, req: Request) -> None:
        """Publish hashes of blocks that became full and computed."""
        if not self.enable_prefix_caching:
            return
        hashes = self.block_hashes(req, req.num_computed_tokens)
        for i, h in enumerate(hashes):
            bid = req.block_ids[i]
            if self.hash_of[bid] is None and h not in self.block_of_hash:
                self.hash_of[bid] = h
                self.block_of_hash[h] = bid


class KVCacheManager:
    """Per-request block bookkeeping on top of a ``BlockPool``."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = False):
        self.pool = BlockPool(num_blocks, block_size, enable_prefix_caching)
        self.block_size = block_size

    @property
    def enable_prefix_caching(self) -> bool:
        return self.pool.enable_prefix_caching

    def reset_prefix_cache(self) -> None:
        self.pool.reset_prefix_cache()

    def blocks_needed(self, req: Request, num_new_tokens: int) -> int:
        total = req.num_computed_tokens + num_new_tokens
        need = (total + self.block_size - 1) // self.block_size
        return max(0, need - len(req.block_ids))

    def can_allocate(self, req: Request, num_new_tokens: int) -> bool:
        return self.blocks_needed(req, num_new_tokens) <= self.pool.num_free

    def allocate(self, req: Request, num_new_tokens: int) -> None:
        n = self.blocks_needed(req, num_new_tokens)
        if n:
            req.block_ids.extend(self.pool.allocate(n))

    def try_prefix_hit(self, req: Request) -> int:
        """Attach cached prefix blocks to a fresh request; returns number of cached tokens."""
        if req.block_ids or req.num_computed_tokens:
            return 0
        hit = self.pool.match_prefix(req)
        if hit:
            req.block_ids = hit
            req.num_computed_tokens = len(hit) * self.block_size
            req.num_cached_tokens = req.num_computed_tokens
        return req.num_computed_tokens

    def commit(self, req: Request) -> None:
        self.pool.register_full_blocks(req)

    def free(self, req: Request) -> None:
        self.pool.release(req.block_ids)
        req.block_ids = []
        for hook in getattr(self, "on_free", ()):     # e.g. the runner's recurrent-state slots
            hook(req)

    @property
    def num_free_blocks(self) -> int:
        return self.pool.num_free

    @property
    def usage(self) -> float:
        return 1.0 - self.pool.num_free / max(self.pool.num_blocks, 1)
