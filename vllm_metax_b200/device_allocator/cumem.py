"""Sleep mode: release the physical memory behind tagged allocations and bring it back at the same
addresses (RLHF co-location: a trainer borrows the GPU between generation phases).

``CuMemAllocator.use_memory_pool(tag)`` routes PyTorch allocations made inside the context through
the native VMM allocator (``csrc/cumem_allocator.cpp``).  ``sleep(offload_tags)`` copies allocations
whose tag is in ``offload_tags`` to pinned host memory and releases the physical memory of ALL pool
allocations (others, e.g. the KV cache, are simply discarded).  ``wake_up(tags)`` re-creates physical
memory at the same virtual addresses and copies the saved bytes back, so every tensor, CUDA graph and
kernel argument that referenced the old memory stays valid.

Parity: vllm_metax/device_allocator/cumem.py:85-316 (CuMemAllocator.get_instance / sleep / wake_up /
use_memory_pool / get_current_usage), patch/enhancement/device_allocator.py:15-19.
"""
from __future__ import annotations

import contextlib
import importlib.util
import threading
from pathlib import Path
from typing import Iterable, Optional

import torch

_native = None
_native_lock = threading.Lock()


def _load_native():
    """Import the in-tree ``_b200_cumem`` extension, building it when the source is newer."""
    global _native
    with _native_lock:
        if _native is not None:
            return _native
        from .. import _build

        lib = _build.build_cumem()
        if lib is None or not Path(lib).exists():
            raise RuntimeError("cumem allocator extension is not built")
        spec = importlib.util.spec_from_file_location("_b200_cumem", str(lib))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.__lib_path__ = str(lib)
        _native = mod
        return mod


class CuMemAllocator:
    _instance: Optional["CuMemAllocator"] = None
    default_tag = "default"

    @staticmethod
    def get_instance() -> "CuMemAllocator":
        if CuMemAllocator._instance is None:
            CuMemAllocator._instance = CuMemAllocator()
        return CuMemAllocator._instance

    def __init__(self, fake_driver: bool = False):
        self.native = _load_native()
        if fake_driver:
            self.native.use_fake_driver(True)
        self.fake = fake_driver
        self._saved: dict[int, torch.Tensor] = {}        # ptr -> pinned host copy
        self._pool = None
        self._pluggable = None
        self.sleeping = False

    # ------------------------------------------------------------------ pool plumbing
    def _torch_pool(self):
        if self._pool is None:
            path = self.native.__lib_path__
            self._pluggable = torch.cuda.memory.CUDAPluggableAllocator(path, "b200_cumem_malloc", "b200_cumem_free")
            self._pool = torch.cuda.memory.MemPool(self._pluggable._allocator)
        return self._pool

    @contextlib.contextmanager
    def use_memory_pool(self, tag: Optional[str] = None):
        """Allocations made by PyTorch inside this context come from the VMM allocator with ``tag``."""
        tag = tag or self.default_tag
        prev = self.native.get_tag()
        self.native.set_tag(tag)
        try:
            if self.fake or not torch.cuda.is_available():
                yield
            else:
                with torch.cuda.use_mem_pool(self._torch_pool()):
                    yield
        finally:
            self.native.set_tag(prev)

    # ------------------------------------------------------------------ raw allocations (tests / fake driver)
    def alloc(self, nbytes: int, device: int = 0, tag: Optional[str] = None) -> int:
        prev = self.native.get_tag()
        self.native.set_tag(tag or prev)
        try:
            return self.native.alloc(nbytes, device)
        finally:
            self.native.set_tag(prev)

    def free(self, ptr: int) -> None:
        self._saved.pop(ptr, None)
        self.native.free(ptr)

    # ------------------------------------------------------------------ copy helpers
    def _to_host(self, ptr: int, size: int, device: int) -> torch.Tensor:
        host = torch.empty(size, dtype=torch.uint8, pin_memory=not self.fake and torch.cuda.is_available())
        with self._device(device):
            self.native.copy(ptr, host.data_ptr(), size, True)
        return host

    def _to_device(self, ptr: int, host: torch.Tensor, device: int) -> None:
        with self._device(device):
            self.native.copy(ptr, host.data_ptr(), host.numel(), False)

    def _device(self, device: int):
        if self.fake or not torch.cuda.is_available():
            return contextlib.nullcontext()
        return torch.cuda.device(device)

    # ------------------------------------------------------------------ sleep / wake
    def sleep(self, offload_tags: Optional[Iterable[str] | str] = None) -> None:
        """Release all pool memory; contents of allocations tagged in ``offload_tags`` survive on the host."""
        if offload_tags is None:
            offload_tags = (self.default_tag,)
        elif isinstance(offload_tags, str):
            offload_tags = (offload_tags,)
        keep = set(offload_tags)
        if not self.fake and torch.cuda.is_available():
            torch.cuda.synchronize()
        for ptr, size, device, tag, mapped in self.native.allocations():
            if not mapped:
                continue
            if tag in keep:
                self._saved[ptr] = self._to_host(ptr, size, device)
            self.native.release(ptr)
        self.sleeping = True
        if not self.fake and torch.cuda.is_available():
            torch.cuda.empty_cache()

    def wake_up(self, tags: Optional[list[str]] = None) -> None:
        """Re-back allocations (all, or those tagged in ``tags``) and restore saved contents."""
        for ptr, size, device, tag, mapped in self.native.allocations():
            if mapped or (tags is not None and tag not in tags):
                continue
            self.native.restore(ptr)
            host = self._saved.pop(ptr, None)
            if host is not None:
                self._to_device(ptr, host, device)
        self.sleeping = any(not m for *_, m in self.native.allocations())

    def get_current_usage(self) -> int:
        """Bytes of physical device memory currently mapped through this allocator."""
        return int(self.native.stats()["mapped_bytes"])

    def stats(self) -> dict:
        return dict(self.native.stats())


def get_mem_allocator_instance() -> CuMemAllocator:
    return CuMemAllocator.get_instance()
