"""KV blocks over TCP between engines on different hosts (or processes): the prefill engine keeps the blocks of the
prompts it has processed in host memory and serves them; the decode engine asks which blocks of a prompt exist and
pulls them.

    producer:  {"kv_connector": "NetworkKVConnector", "kv_role": "kv_producer",
                "kv_connector_extra_config": {"listen": "0.0.0.0:14579", "max_bytes": 8 << 30}}
    consumer:  {"kv_connector": "NetworkKVConnector", "kv_role": "kv_consumer",
                "kv_connector_extra_config": {"peers": ["10.0.0.5:14579"]}}

Blocks are addressed by the chained hash of the tokens up to and including them (any shared prefix is found) and
travel as ``crc32 | length | bytes of every cache tensor's slice``; a block that is missing, short or fails its
checksum ends the load there and the scheduler recomputes the rest.  The store is bounded (least recently used
blocks are dropped).  Requests: ``H`` + n hashes -> n availability bytes; ``G`` + one hash -> the blob (empty = miss).
This is the role of the network connectors the reference inherits from upstream (P2P-NCCL / Mooncake / NIXL in its
disaggregated-serving examples, examples/disaggregated/* in its tree), with host-staged TCP as the transport.
"""
from __future__ import annotations

import collections
import socket
import socketserver
import struct
import threading
from typing import Optional

from .base import KVConnector, KVTransferConfig
from .shared_storage import SharedStorageConnector, chain_hashes

HASH_BYTES = 40


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(1 << 20, n - len(buf)))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return bytes(buf)


class BlockStore:
    """hash -> blob, bounded, least recently used out first; shared by the server threads and the engine thread."""

    def __init__(self, max_bytes: int):
        self.max_bytes = max_bytes
        self.size = 0
        self.blobs: "collections.OrderedDict[str, bytes]" = collections.OrderedDict()
        self.lock = threading.Lock()

    def put(self, h: str, blob: bytes) -> bool:
        with self.lock:
            if h in self.blobs:
                self.blobs.move_to_end(h)
                return False
            self.blobs[h] = blob
            self.size += len(blob)
            while self.size > self.max_bytes and len(self.blobs) > 1:
                _, old = self.blobs.popitem(last=False)
                self.size -= len(old)
            return True

    def get(self, h: str) -> Optional[bytes]:
        with self.lock:
            b = self.blobs.get(h)
            if b is not None:
                self.blobs.move_to_end(h)
            return b

    def has(self, h: str) -> bool:
        with self.lock:
            return h in self.blobs


class _Handler(socketserver.BaseRequestHandler):
    def handle(self) -> None:
        store: BlockStore = self.server.store           # type: ignore[attr-defined]
        sock = self.request
        try:
            while True:
                op = sock.recv(1)
                if not op:
                    return
                if op == b"H":
                    (n,) = struct.unpack("<I", _recv_exact(sock, 4))
                    raw = _recv_exact(sock, n * HASH_BYTES)
                    sock.sendall(bytes(1 if store.has(raw[i * HASH_BYTES:(i + 1) * HASH_BYTES].decode()) else 0
                                       for i in range(n)))
                elif op == b"G":
                    blob = store.get(_recv_exact(sock, HASH_BYTES).decode()) or b""
                    sock.sendall(struct.pack("<Q", len(blob)) + blob)
                else:
                    return
        except (ConnectionError, OSError):
            return


class _Server(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True


class NetworkKVConnector(SharedStorageConnector):
    """Same block format as the shared-storage connector; the blocks live in the producer's memory and cross TCP."""

    def __init__(self, config: KVTransferConfig, runner):
        KVConnector.__init__(self, config, runner)
        extra = config.kv_connector_extra_config
        self.block_size = runner.block_size
        if not self._tensors():
            raise NotImplementedError("no paged cache tensors found on the runner")
        self.timeout = float(extra.get("timeout_s", 10.0))
        self.store = BlockStore(int(extra.get("max_bytes", 4 << 30)))
        self.server = None
        self.address = None
        if config.is_producer:
            host, _, port = str(extra.get("listen", "127.0.0.1:0")).rpartition(":")
            self.server = _Server((host or "127.0.0.1", int(port or 0)), _Handler)
            self.server.store = self.store
            self.address = "%s:%d" % self.server.server_address[:2]
            threading.Thread(target=self.server.serve_forever, name="b200-kv-server", daemon=True).start()
        self.peers = [str(p) for p in extra.get("peers", [])]
        self._socks: dict = {}
        self.stats.update(bytes_sent=0, bytes_received=0)

    # ------------------------------------------------------------------ client side
    def _sock(self, peer: str) -> socket.socket:
        s = self._socks.get(peer)
        if s is None:
            host, _, port = peer.rpartition(":")
            s = socket.create_connection((host, int(port)), timeout=self.timeout)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            self._socks[peer] = s
        return s

    def _drop(self, peer: str) -> None:
        s = self._socks.pop(peer, None)
        if s is not None:
            try:
                s.close()
            except OSError:
                pass

    def _has(self, peer: str, hashes: list) -> list:
        try:
            s = self._sock(peer)
            s.sendall(b"H" + struct.pack("<I", len(hashes)) + "".join(hashes).encode())
            return [b == 1 for b in _recv_exact(s, len(hashes))]
        except (OSError, ConnectionError):
            self._drop(peer)
            return [False] * len(hashes)

    def _get(self, peer: str, h: str) -> Optional[bytes]:
        try:
            s = self._sock(peer)
            s.sendall(b"G" + h.encode())
            (n,) = struct.unpack("<Q", _recv_exact(s, 8))
            blob = _recv_exact(s, n) if n else b""
            self.stats["bytes_received"] += n
            return blob or None
        except (OSError, ConnectionError):
            self._drop(peer)
            return None

    # ------------------------------------------------------------------ interface
    def lookup(self, token_ids: list, salt=None) -> int:
        hs = chain_hashes(token_ids, self.block_size, salt)
        if not hs:
            return 0
        best = 0
        local = [self.store.has(h) for h in hs]
        for have in [local] + [self._has(p, hs) for p in self.peers]:
            n = next((i for i, ok in enumerate(have) if not ok), len(have))
            best = max(best, n)
        return best * self.block_size

    def load(self, token_ids: list, block_ids: list, num_tokens: int, salt=None, first_block: int = 0) -> int:
        hs = chain_hashes(token_ids[:num_tokens], self.block_size, salt)
        done = first_block * self.block_size
        for h, bid in list(zip(hs, block_ids))[first_block:]:
            blob = self.store.get(h)
            for p in self.peers:
                if blob is not None:
                    break
                blob = self._get(p, h)
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
            blob = self._pack(bid)
            if self.store.put(h, blob):
                wrote += 1
                self.stats["bytes_sent"] += 0          # counted when a peer pulls; kept for symmetry of the stats
        self.stats["blocks_saved"] += wrote
        return wrote

    def close(self) -> None:
        for p in list(self._socks):
            self._drop(p)
        if self.server is not None:
            self.server.shutdown()
            self.server.server_close()
            self.server = None
