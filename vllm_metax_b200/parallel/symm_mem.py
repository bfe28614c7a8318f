"""Symmetric (peer-mapped) device memory for in-kernel NVLink collectives.

Every rank of a group allocates one buffer with ``cudaMalloc``, exports its CUDA-IPC handle,
and opens the handles of all peers (exchanged as 64-byte blobs over the group's Gloo/CPU
process group).  The result is a table ``ptrs[r]`` of device addresses valid on THIS rank for
rank r's buffer; kernels store to / load from those addresses directly over NVLink.

Regions of the buffer are carved with ``region()`` at identical offsets on all ranks (hence
"symmetric"), so ``peer_ptrs(region)`` is just base addresses plus one offset.

Parity: the reference builds the same thing for its only in-kernel collective -
``IpcBuffer`` / ``LamportWorkspace`` (vllm_metax/registry/custom_ops/layers/minimax_rms_norm/
lamport_workspace.py:53-232: fine-grained malloc, cudaIpcGetMemHandle, all_gather_object,
cudaIpcOpenMemHandle, device pointer table).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _custom_ops as ops
from .state import Group


@dataclass
class Region:
    name: str
    offset: int
    nbytes: int


class SymmWorkspace:
    ALIGN = 1024

    def __init__(self, group: Group, nbytes: int, device: torch.device):
        assert device.type == "cuda"
        ops.load_native()
        self.group = group
        self.device = device
        self.world = group.world_size
        self.rank = group.rank_in_group
        self.nbytes = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        dev_index = device.index if device.index is not None else torch.cuda.current_device()
        self.buffer, handle = torch.ops.b200.symm_alloc(self.nbytes, dev_index)
        blobs = group.all_gather_object(bytes(handle.numpy().tobytes()))
        self.base_ptrs: list[int] = []
        self._opened: list[int] = []
        for r, blob in enumerate(blobs):
            if r == self.rank:
                self.base_ptrs.append(self.buffer.data_ptr())
            else:
                h = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
                ptr = int(torch.ops.b200.symm_open(h, dev_index))
                self._opened.append(ptr)
                self.base_ptrs.append(ptr)
        self._cursor = 0
        self.regions: dict[str, Region] = {}
        group.barrier()

    def region(self, name: str, nbytes: int) -> Region:
        if name in self.regions:
            return self.regions[name]
        off = (self._cursor + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if off + nbytes > self.nbytes:
            raise RuntimeError(f"symmetric workspace exhausted: {name} needs {nbytes} bytes at {off} of {self.nbytes}")
        self._cursor = off + nbytes
        r = Region(name, off, nbytes)
        self.regions[name] = r
        return r

    def local(self, region: Region, dtype: torch.dtype, shape) -> torch.Tensor:
        """This rank's copy of the region as a tensor."""
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty((), dtype=dtype).element_size()
        assert n * esz <= region.nbytes
        return self.buffer[region.offset: region.offset + n * esz].view(dtype).view(*shape)

    def peer_ptrs(self, region: Region) -> list[int]:
        return [b + region.offset for b in self.base_ptrs]

    def close(self) -> None:
        for p in self._opened:
            torch.ops.b200.symm_close(p)
        self._opened = []
        self.buffer = None
