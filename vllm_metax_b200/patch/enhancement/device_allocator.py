"""Route vLLM's sleep-mode allocator lookup to this package's VMM allocator.
Parity: vllm_metax/patch/enhancement/device_allocator.py:15-19."""
from .. import utils


@utils.patch("vllm.device_allocator", "get_mem_allocator_instance", allow_new=True)
def get_mem_allocator_instance():
    from ...device_allocator.cumem import CuMemAllocator

    return CuMemAllocator.get_instance()
