"""Host-side failure detection between the ranks of one engine.

Every rank runs the same scheduler in lock step, so a rank whose step raised must tell the others before they
launch kernels that would wait for it.  This is done on the host, through the key-value store the process groups
were built on:

* ``announce_failure(reason)`` - called from the failing rank's exception handler; writes ``dead/<rank>``.
* ``check()`` - called by every rank before it launches a step; raises ``PeerFailedError`` naming the first dead
  peer.  No GPU work is in flight at that point, so the rank can release its memory and stop cleanly.
* ``beat(step)`` / ``stale_peers(max_age_s)`` - a heartbeat for peers that died without running their handler
  (killed process): a rank whose last beat is older than ``max_age_s`` is reported.

A peer that fails while the others already sit inside a collective is caught by the process-group timeout
(``B200_PG_TIMEOUT_S``) or, inside this package's own kernels, by the bounded flag waits.
Parity: upstream's worker-death handling that turns any rank failure into ``EngineDeadError`` for all callers
(tests/v1/shutdown/test_forward_error.py:21-80 in the reference tree).
"""
from __future__ import annotations

import time
from typing import Optional


class PeerFailedError(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class RankLiveness:
    def __init__(self, store, rank: int, world: int, prefix: str = "b200_live"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    @classmethod
    def from_default_group(cls, prefix: str = "b200_live") -> Optional["RankLiveness"]:
        """Built on the store of the default process group; ``None`` in a single-process run."""
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return None
        from torch.distributed.distributed_c10d import _get_default_store

        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), prefix)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def announce_failure(self, reason: str) -> None:
        try:
            self.store.set(self._key("dead", self.rank), reason[:500])
        except Exception:      # the store host may be the rank that died
            pass

    def beat(self, step: int) -> None:
        self.store.set(self._key("beat", self.rank), f"{step}:{time.time():.3f}")

    def check(self) -> None:
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key("dead", r)]):
                raise PeerFailedError(r, self.store.get(self._key("dead", r)).decode(errors="replace"))

    def stale_peers(self, max_age_s: float) -> list[int]:
        now, out = time.time(), []
        for r in range(self.world):
            if r == self.rank or not self.store.check([self._key("beat", r)]):
                continue
            ts = float(self.store.get(self._key("beat", r)).decode().split(":")[1])
            if now - ts > max_age_s:
                out.append(r)
        return out
