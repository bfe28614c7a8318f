"""Sleep-mode allocator: bookkeeping round trip against the host-memory fake of the driver (CPU), and the
real VMM path on a GPU (tensor contents and addresses survive sleep / wake)."""
import ctypes

import pytest
import torch

from vllm_metax_b200.device_allocator.cumem import CuMemAllocator

gpu = pytest.mark.gpu


def test_sleep_wake_roundtrip_fake_driver():
    alloc = CuMemAllocator(fake_driver=True)
    try:
        w = alloc.alloc(3 << 20, 0, tag="weights")
        kv = alloc.alloc(5 << 20, 0, tag="kv_cache")
        payload = bytes(range(256)) * 16
        ctypes.memmove(w, payload, len(payload))
        assert alloc.get_current_usage() == (4 << 20) + (6 << 20)      # padded to the 2 MiB granularity
        alloc.sleep(offload_tags=("weights",))
        assert alloc.get_current_usage() == 0 and alloc.sleeping
        tags = {t: m for _, _, _, t, m in alloc.native.allocations()}
        assert tags == {"weights": False, "kv_cache": False}
        alloc.wake_up(tags=["weights"])
        assert alloc.get_current_usage() == 4 << 20 and alloc.sleeping   # kv cache still released
        assert ctypes.string_at(w, len(payload)) == payload
        alloc.wake_up()
        assert alloc.get_current_usage() == 10 << 20 and not alloc.sleeping
        alloc.free(w)
        alloc.free(kv)
        assert alloc.stats()["allocations"] == 0
    finally:
        alloc.native.use_fake_driver(False)


def test_free_unknown_pointer_raises():
    alloc = CuMemAllocator(fake_driver=True)
    try:
        with pytest.raises(RuntimeError):
            alloc.native.free(12345)
    finally:
        alloc.native.use_fake_driver(False)


@gpu
def test_sleep_wake_gpu():
    alloc = CuMemAllocator.get_instance()
    with alloc.use_memory_pool("weights"):
        w = torch.arange(1 << 20, device="cuda", dtype=torch.float32)
    with alloc.use_memory_pool("kv_cache"):
        kv = torch.ones(4 << 20, device="cuda", dtype=torch.bfloat16)
    ptr = w.data_ptr()
    used = alloc.get_current_usage()
    assert used >= w.numel() * 4 + kv.numel() * 2
    free0 = torch.cuda.mem_get_info()[0]
    alloc.sleep(offload_tags="weights")
    assert alloc.get_current_usage() == 0
    assert torch.cuda.mem_get_info()[0] >= free0 + used // 2
    alloc.wake_up()
    assert w.data_ptr() == ptr and alloc.get_current_usage() == used
    assert torch.equal(w.cpu(), torch.arange(1 << 20, dtype=torch.float32))
    kv.fill_(2.0)                     # discarded contents, but the memory is usable again
    assert float(kv[-1]) == 2.0
    del w, kv
