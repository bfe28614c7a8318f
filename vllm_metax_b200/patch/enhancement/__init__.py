"""Compatibility features layered onto upstream vLLM."""
from . import bench_serve_args, device_allocator, fp8_block_kernel, int8_quantize  # noqa: F401
