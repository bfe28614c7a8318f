"""One file per KV block in a directory both engines can reach (tmpfs, a shared file system)."""
from __future__ import annotations

import hashlib
import os
import struct
import zlib
from typing import Optional

import torch

from .base import KVConnector, KVTransferConfig


def chain_hashes(token_ids: list, block_size: int, salt=None) -> list[str]:
    """Process-independent chained hashes of the full blocks of ``token_ids``."""
    out, parent = [], hashlib.sha256(repr(salt).encode()).digest()
    for i in range(len(token_ids) // block_size):
        blk = token_ids[i * block_size:(i + 1) * block_size]
        parent = hashlib.sha256(parent + struct.pack(f"<{block_size}q", *blk)).digest()
        out.append(parent.hex()[:40])
    return out


class SharedStorageConnector(KVConnector):
    def __init__(self, config: KVTransferConfig, runner):
        super().__init__(config, runner)
        self.path = config.kv_connector_extra_config.get("shared_storage_path", "/tmp/b200_kv_store")
        os.makedirs(self.path, exist_ok=True)
        self.block_size = runner.block_size
        if not self._tensors():
            raise NotImplementedError("no paged cache tensors found on the runner")

    def _tensors(self) -> list:
        """Every per-layer tensor whose leading dimension is the block index (caches and their scale planes)."""
        out = []
        for entry in self.runner.kv_caches:
            for t in (entry if isinstance(entry, (tuple, list)) else (entry,)):
                if torch.is_tensor(t) and t.dim() >= 2:
                    out.append(t)
        return out

    def _file(self, h: str) -> str:
        return os.path.join(self.path, h + ".kv")

    # ------------------------------------------------------------------ one block <-> bytes
    def _pack(self, bid: int) -> bytes:
        body = b"".join(t[bid].contiguous().view(torch.uint8).cpu().numpy().tobytes() for t in self._tensors())
        return struct.pack("<IQ", zlib.crc32(body), len(body)) + body

    def _unpack(self, bid: int, blob: bytes) -> bool:
        if len(blob) < 12:
            return False
        crc, n = struct.unpack("<IQ", blob[:12])
        body = blob[12:]
        if len(body) != n or zlib.crc32(body) != crc:
            return False
        off = 0
        views = []
        for t in self._tensors():
            nb = t[bid].numel() * t.element_size()
            if off + nb > n:
                return False
            views.append((t, off, nb))
            off += nb
        if off != n:
            return False                                   # written by an engine with another cache geometry
        for t, o, nb in views:
            src = torch.frombuffer(bytearray(body[o:o + nb]), dtype=torch.uint8)
            t[bid].view(torch.uint8).reshape(-1).copy_(src.to(t.device))
        return True

    # ------------------------------------------------------------------ interface
    def lookup(self, token_ids: list, salt=None) -> int:
        n = 0
        for h in chain_hashes(token_ids, self.block_size, salt):
            if not os.path.exists(self._file(h)):
                break
            n += self.block_size
        return n

    def load(self, token_ids: list, block_ids: list, num_tokens: int, salt=None, first_block: int = 0) -> int:
        hs = chain_hashes(token_ids[:num_tokens], self.block_size, salt)
        done = first_block * self.block_size               # blocks before first_block are already in the cache
        for h, bid in list(zip(hs, block_ids))[first_block:]:
            try:
                with open(self._file(h), "rb") as f:
                    ok = self._unpack(bid, f.read())
            except OSError:
                ok = False
            if not ok:
                self.stats["load_failures"] += 1
                break
            done += self.block_size
            self.stats["blocks_loaded"] += 1
        return done

    def save(self, token_ids: list, block_ids: list, num_tokens: int, salt=None) -> int:
        hs = chain_hashes(token_ids[:num_tokens], self.block_size, salt)
        wrote = 0
        for h, bid in zip(hs, block_ids):
            fn = self._file(h)
            if os.path.exists(fn):
                continue
            tmp = f"{fn}.{os.getpid()}.tmp"
            with open(tmp, "wb") as f:
                f.write(self._pack(bid))
            os.replace(tmp, fn)                            # readers never see a half-written block
            wrote += 1
        self.stats["blocks_saved"] += wrote
        return wrote
