"""Patches that only change speed."""
from . import grouped_topk_router, speculative_decode_perf, unquantized_gemm  # noqa: F401
