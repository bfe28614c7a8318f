"""Read-only NVML queries (device identity, memory, NVLink topology, NUMA node, clocks).

Everything here READS device state; nothing sets clocks, power limits or modes.  The backend module
is injectable (``set_backend``) so the logic runs in CPU tests against a fake NVML.

Parity: the mxsml-based queries of vllm_metax/platform.py:707-906 (``with_mxsml_context``, name /
uuid / total memory / ``is_fully_connected`` over MetaXLink / NUMA node / PCI bus ids) and the
thin ctypes shim vllm_metax/utils/mxsml.py.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Any, Iterator, Optional

_backend: Any = None
_lock = threading.RLock()
_depth = 0


def set_backend(module: Any) -> None:
    """Use ``module`` (pynvml-compatible API) instead of the real pynvml.  ``None`` restores it."""
    global _backend
    _backend = module


def _module():
    if _backend is not None:
        return _backend
    import pynvml  # provided by nvidia-ml-py

    return pynvml


def _s(x) -> str:
    return x.decode() if isinstance(x, bytes) else str(x)


class NvmlSession:
    def __init__(self, mod):
        self.m = mod

    def device_count(self) -> int:
        return int(self.m.nvmlDeviceGetCount())

    def _h(self, idx: int):
        return self.m.nvmlDeviceGetHandleByIndex(idx)

    def device_name(self, idx: int) -> str:
        return _s(self.m.nvmlDeviceGetName(self._h(idx)))

    def device_uuid(self, idx: int) -> str:
        return _s(self.m.nvmlDeviceGetUUID(self._h(idx)))

    def device_capability(self, idx: int) -> tuple[int, int]:
        major, minor = self.m.nvmlDeviceGetCudaComputeCapability(self._h(idx))
        return int(major), int(minor)

    def device_memory_total(self, idx: int) -> int:
        return int(self.m.nvmlDeviceGetMemoryInfo(self._h(idx)).total)

    def device_memory_used(self, idx: int) -> int:
        return int(self.m.nvmlDeviceGetMemoryInfo(self._h(idx)).used)

    def device_pci_bus_id(self, idx: int) -> str:
        return _s(self.m.nvmlDeviceGetPciInfo(self._h(idx)).busId)

    def device_numa_node(self, idx: int) -> Optional[int]:
        fn = getattr(self.m, "nvmlDeviceGetNumaNodeId", None)
        if fn is not None:
            try:
                return int(fn(self._h(idx)))
            except Exception:
                pass
        # sysfs fallback keyed by the PCI address
        try:
            bus = self.device_pci_bus_id(idx).lower()
            if len(bus.split(":")[0]) == 8:   # NVML pads the domain to 8 hex digits; sysfs uses 4
                bus = bus[4:]
            with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
                node = int(f.read().strip())
            return node if node >= 0 else None
        except Exception:
            return None

    def clocks(self, idx: int) -> dict[str, int]:
        h = self._h(idx)
        m = self.m
        return {
            "sm_mhz": int(m.nvmlDeviceGetClockInfo(h, m.NVML_CLOCK_SM)),
            "sm_max_mhz": int(m.nvmlDeviceGetMaxClockInfo(h, m.NVML_CLOCK_SM)),
            "mem_mhz": int(m.nvmlDeviceGetClockInfo(h, m.NVML_CLOCK_MEM)),
        }

    def power_watts(self, idx: int) -> float:
        return self.m.nvmlDeviceGetPowerUsage(self._h(idx)) / 1000.0

    def nvlink_active_links(self, idx: int) -> int:
        h = self._h(idx)
        n = 0
        for link in range(int(getattr(self.m, "NVML_NVLINK_MAX_LINKS", 18))):
            try:
                if self.m.nvmlDeviceGetNvLinkState(h, link):
                    n += 1
            except Exception:
                break
        return n

    def p2p_ok(self, a: int, b: int) -> bool:
        """True when NVLink peer access between a and b is reported OK."""
        m = self.m
        try:
            st = m.nvmlDeviceGetP2PStatus(self._h(a), self._h(b), m.NVML_P2P_CAPS_INDEX_NVLINK)
            return st == m.NVML_P2P_STATUS_OK
        except Exception:
            return False

    def fully_connected(self, ids: list[int]) -> bool:
        """Every pair of ``ids`` reaches each other over NVLink (directly or through NVSwitch)."""
        for i, a in enumerate(ids):
            for b in ids[i + 1:]:
                if not self.p2p_ok(a, b):
                    return False
        return True

    def summary(self) -> list[dict[str, Any]]:
        out = []
        for i in range(self.device_count()):
            out.append({
                "index": i, "name": self.device_name(i), "uuid": self.device_uuid(i),
                "memory_total": self.device_memory_total(i), "pci": self.device_pci_bus_id(i),
                "numa": self.device_numa_node(i), "nvlinks": self.nvlink_active_links(i),
            })
        return out


@contextlib.contextmanager
def session() -> Iterator[NvmlSession]:
    """``nvmlInit`` on first entry, ``nvmlShutdown`` when the outermost context exits."""
    global _depth
    mod = _module()
    with _lock:
        if _depth == 0:
            mod.nvmlInit()
        _depth += 1
    try:
        yield NvmlSession(mod)
    finally:
        with _lock:
            _depth -= 1
            if _depth == 0:
                try:
                    mod.nvmlShutdown()
                except Exception:
                    pass
