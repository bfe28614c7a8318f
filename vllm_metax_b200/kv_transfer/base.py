from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class KVTransferConfig:
    kv_connector: str = "SharedStorageConnector"
    kv_role: str = "kv_both"                     # kv_producer | kv_consumer | kv_both
    kv_connector_extra_config: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["KVTransferConfig"]:
        if not d:
            return None
        c = cls(**{k: v for k, v in d.items() if k in ("kv_connector", "kv_role", "kv_connector_extra_config")})
        if c.kv_role not in ("kv_producer", "kv_consumer", "kv_both"):
            raise ValueError(f"unknown kv_role {c.kv_role!r}")
        return c

    @property
    def is_producer(self) -> bool:
        return self.kv_role in ("kv_producer", "kv_both")

    @property
    def is_consumer(self) -> bool:
        return self.kv_role in ("kv_consumer", "kv_both")


class KVConnector:
    """What the engine calls.  Token counts are multiples of the cache block size."""

    def __init__(self, config: KVTransferConfig, runner):
        self.config, self.runner = config, runner
        self.stats = {"blocks_saved": 0, "blocks_loaded": 0, "load_failures": 0}

    def lookup(self, token_ids: list, salt=None) -> int:
        """Leading tokens of ``token_ids`` whose KV is available outside this engine."""
        raise NotImplementedError

    def load(self, token_ids: list, block_ids: list, num_tokens: int, salt=None, first_block: int = 0) -> int:
        """Fill ``block_ids[first_block:]`` with the KV of the first ``num_tokens`` tokens; returns the length of the
        valid prefix (less than asked when a block is missing or corrupt - the caller recomputes the rest)."""
        raise NotImplementedError

    def save(self, token_ids: list, block_ids: list, num_tokens: int, salt=None) -> int:
        """Publish the KV of the first ``num_tokens`` tokens; returns the number of blocks written."""
        raise NotImplementedError


def make_connector(config: Optional[KVTransferConfig], runner) -> Optional[KVConnector]:
    if config is None:
        return None
    from .host_offload import HostOffloadConnector
    from .network import NetworkKVConnector
    from .shared_storage import SharedStorageConnector

    kinds = {"SharedStorageConnector": SharedStorageConnector, "NetworkKVConnector": NetworkKVConnector,
             "P2pNcclConnector": NetworkKVConnector,      # upstream's name for "pull blocks from the prefill engine"
             "OffloadingConnector": HostOffloadConnector, "HostOffloadConnector": HostOffloadConnector}
    if config.kv_connector not in kinds:
        raise ValueError(f"unknown kv_connector {config.kv_connector!r}; available: {', '.join(kinds)}")
    return kinds[config.kv_connector](config, runner)
