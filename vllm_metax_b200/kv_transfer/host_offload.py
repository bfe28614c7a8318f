"""Host-memory KV offload tier: one engine keeps the KV blocks of the prompts it has processed in (bounded, LRU) host
memory and attaches them again when a later request shares the prefix - after the device-side prefix cache has long
evicted them, or with the device-side cache switched off.

    LLM(model, kv_transfer_config={"kv_connector": "OffloadingConnector", "kv_role": "kv_both",
                                   "kv_connector_extra_config": {"cpu_bytes_to_use": 64 << 30}})

Blocks are addressed by the chained hash of the tokens up to and including the block (as in the other connectors), so
any shared prefix hits; a block that was evicted from host memory, or whose checksum fails, ends the load there and the
rest of the prompt is computed.  The same store and record format as the network connector, without the network.
Parity: upstream's CPU offloading connector / the LMCache examples the reference ships
(examples/disaggregated/*lmcache* in its tree) for the single-engine "extend the prefix cache into host memory" use.
"""
from __future__ import annotations

from .base import KVTransferConfig
from .network import BlockStore
from .shared_storage import SharedStorageConnector, chain_hashes


class HostOffloadConnector(SharedStorageConnector):
    def __init__(self, config: KVTransferConfig, runner):
        extra = dict(config.kv_connector_extra_config)
        extra.setdefault("shared_storage_path", "/tmp/b200_kv_store_unused")
        super().__init__(KVTransferConfig(config.kv_connector, config.kv_role, extra), runner)
        self.config = config
        self.store = BlockStore(int(extra.get("cpu_bytes_to_use", extra.get("max_bytes", 8 << 30))))

    def lookup(self, token_ids: list, salt=None) -> int:
        n = 0
        for h in chain_hashes(token_ids, self.block_size, salt):
            if not self.store.has(h):
                break
            n += self.block_size
        return n

    def load(self, token_ids: list, block_ids: list, num_tokens: int, salt=None, first_block: int = 0) -> int:
        hs = chain_hashes(token_ids[:num_tokens], self.block_size, salt)
        done = first_block * self.block_size
        for h, bid in list(zip(hs, block_ids))[first_block:]:
            blob = self.store.get(h)
            if blob is None or not self._unpack(bid, blob):
                self.stats["load_failures"] += 1
                break
            done += self.block_size
            self.stats["blocks_loaded"] += 1
        return done

    def save(self, token_ids: list, block_ids: list, num_tokens: int, salt=None) -> int:
        hs = chain_hashes(token_ids[:num_tokens], self.block_size, salt)
        wrote = 0
        for h, bid in zip(hs, block_ids):
            if self.store.has(h):
                continue
            wrote += bool(self.store.put(h, self._pack(bid)))
        self.stats["blocks_saved"] += wrote
        return wrote
