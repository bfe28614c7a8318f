"""KV transfer between engines (disaggregated prefill): a prefill engine publishes the KV blocks of the prompts it
has processed, a decode engine pulls them instead of recomputing the prompt.

    LLM(model, kv_transfer_config={"kv_connector": "SharedStorageConnector", "kv_role": "kv_producer",
                                   "kv_connector_extra_config": {"shared_storage_path": "/dev/shm/kv"}})

``KVConnector`` is the interface; ``NetworkKVConnector`` (``network.py``) serves the blocks from the producer's memory
over TCP; ``HostOffloadConnector`` (``host_offload.py``) is the single-engine form, a host-memory tier behind the
device's prefix cache; ``SharedStorageConnector`` keeps one file per KV block, addressed by the chained
hash of the tokens up to and including that block, so any shared prompt prefix is found.  A block that is missing
or fails its checksum ends the load there: the scheduler recomputes the rest and counts the failure.
Parity: the disaggregated-prefill examples of the reference (examples/disaggregated/* and
kv_load_failure_recovery_offline/README.md:1-30 in its tree) and ``Platform.insert_blocks_to_device`` /
``swap_out_blocks_to_host`` (vllm_metax/platform.py:619-640).
"""
from .base import KVConnector, KVTransferConfig, make_connector
from .host_offload import HostOffloadConnector
from .network import NetworkKVConnector
from .shared_storage import SharedStorageConnector

__all__ = ["HostOffloadConnector", "KVConnector", "KVTransferConfig", "NetworkKVConnector", "SharedStorageConnector",
           "make_connector"]
