"""Environment-variable flag system, evaluated lazily on attribute access.

Every flag is declared once in ``environment_variables`` with a resolver that
parses ``os.environ`` at the moment the attribute is read, so tests and launch
scripts can flip a flag after import.  ``override_env`` rewrites both the
resolver and ``os.environ`` and logs the reason, and can forward the override
to ``vllm.envs`` when vLLM is importable.

Parity: vllm_metax/envs.py:27-109 (table), :113-149 (override_vllm_env),
:152-167 (module ``__getattr__``/``__dir__``).
"""
from __future__ import annotations

import logging
import os
from typing import Any, Callable

logger = logging.getLogger(__name__)


def _flag(name: str, default: str) -> Callable[[], bool]:
    return lambda: os.environ.get(name, default).strip().lower() in ("1", "true", "yes", "on")


def _int(name: str, default: int) -> Callable[[], int]:
    return lambda: int(os.environ.get(name, str(default)))


def _str(name: str, default: str | None) -> Callable[[], str | None]:
    return lambda: os.environ.get(name, default)


environment_variables: dict[str, Callable[[], Any]] = {
    # ---- build time -------------------------------------------------------
    "B200_TARGET_DEVICE": _str("B200_TARGET_DEVICE", "cuda"),
    "MAX_JOBS": _str("MAX_JOBS", None),
    "NVCC_THREADS": _str("NVCC_THREADS", None),
    "CMAKE_BUILD_TYPE": _str("CMAKE_BUILD_TYPE", None),
    "VERBOSE": _flag("VERBOSE", "0"),
    "CUDA_HOME": _str("CUDA_HOME", "/usr/local/cuda"),
    # When 1 the native extension must already be built in-tree; never JIT.
    "B200_USE_PREBUILT_KERNELS": _flag("B200_USE_PREBUILT_KERNELS", "0"),
    # ---- runtime: kernel selection ---------------------------------------
    # Hand-written tcgen05 GEMM on dense linears (0 = cuBLAS, debug only).
    "B200_TCGEN05_GEMM": _flag("B200_TCGEN05_GEMM", "1"),
    # Fused GEMM + in-kernel NVLink all-reduce + residual + RMSNorm.
    "B200_FUSED_TP_COLLECTIVES": _flag("B200_FUSED_TP_COLLECTIVES", "1"),
    # Which fused row-parallel path runs: "split" = GEMM with NVLink row-scatter epilogue + one reduce / norm /
    # all-gather kernel (every step size), "mono" = the single 128x256-tile kernel (steps of at least
    # B200_FUSED_TP_MIN_TOKENS tokens; GEMM + peer-store all-reduce + add-norm below).
    "B200_FUSED_TP_KERNEL": _str("B200_FUSED_TP_KERNEL", "split"),
    "B200_FUSED_TP_MIN_TOKENS": _int("B200_FUSED_TP_MIN_TOKENS", 1024),
    # Cascade attention: requests of a step whose leading cache blocks are the same physical blocks (prefix cache)
    # attend that prefix once for the whole step.  Taken when prefix_tokens * (requests - 1) reaches the threshold.
    "B200_CASCADE_ATTENTION": _flag("B200_CASCADE_ATTENTION", "1"),
    "B200_CASCADE_MIN_SAVED_TOKENS": _int("B200_CASCADE_MIN_SAVED_TOKENS", 131072),
    # Batch-invariant execution (the reference's VLLM_BATCH_INVARIANT, vllm_metax/v1/attention/backends/flash_attn.py:1063,
    # 1145): a request's tokens must not depend on what else is in its step.  Every reduction whose order follows the
    # batch is pinned: decode attention and MLA decode run unsplit, GEMMs take one fixed tile shape without split-K /
    # stream-K / CTA pairs / operand swap, cascade attention and the fused tensor-parallel collectives are off.
    "B200_BATCH_INVARIANT": _flag("B200_BATCH_INVARIANT", "0"),
    # Gated delta rule (Qwen3-Next): prompt chunks of at least MIN_TOKENS tokens take the chunked matrix form
    # (ops/gdn.py:gated_delta_rule_chunked, PyTorch products) instead of the recurrent kernel.  0 = always recurrent.
    "B200_GDN_CHUNKED": _flag("B200_GDN_CHUNKED", "0"),
    "B200_GDN_CHUNKED_MIN_TOKENS": _int("B200_GDN_CHUNKED_MIN_TOKENS", 256),
    # Absorbed-MLA decode on tcgen05 (csrc/mla_decode_tcgen05.cu) for dense 16-bit caches from 64 heads per rank up;
    # 0 = the mma.sync kernel unless a call asks for the tcgen05 one.
    "B200_MLA_TCGEN05": _flag("B200_MLA_TCGEN05", "0"),
    # Prepare step k + 1 on the host (schedule, staging buffers) while the device runs step k; 0 = strictly in turn.
    "B200_OVERLAP_SCHEDULING": _flag("B200_OVERLAP_SCHEDULING", "1"),
    # Pipeline parallel: keep one step per stage in flight (disjoint request sets) instead of running lock-step.
    "B200_PP_OVERLAP": _flag("B200_PP_OVERLAP", "1"),
    # Stream-K CTA-pair GEMM for skinny problems (read by the native GEMM dispatcher; 0 = tile / split-K kernels).
    "B200_GEMM_STREAMK": _flag("B200_GEMM_STREAMK", "1"),
    # One query tile per CTA in the prefill attention kernel (read by the native dispatcher; debug only).
    "B200_ATTN_PREFILL_SINGLE": _flag("B200_ATTN_PREFILL_SINGLE", "0"),
    # Sequence-parallel MoE through the NVLink dispatch / combine kernels instead of experts-on-all-tokens + all-reduce.
    "B200_MOE_A2A": _flag("B200_MOE_A2A", "0"),
    # Pack topk weights/ids/scales into one tensor for the AG/RS dispatch.
    # Tokens per pass through the expert kernels (bounds the expert-sorted workspace of a MoE layer on very long steps;
    # the reference's VLLM_FUSED_MOE_CHUNK_SIZE).  0 = never split.
    "B200_FUSED_MOE_CHUNK_SIZE": _int("B200_FUSED_MOE_CHUNK_SIZE", 32768),
    "B200_OPTIMIZED_DP_ALL2ALL": _flag("B200_OPTIMIZED_DP_ALL2ALL", "1"),
    "B200_SUPPORTS_FP8": _flag("B200_SUPPORTS_FP8", "1"),
    "B200_USE_FUSED_GROUPED_TOPK": _flag("B200_USE_FUSED_GROUPED_TOPK", "1"),
    # CUDA-graph capture of decode steps.
    "B200_CUDA_GRAPHS": _flag("B200_CUDA_GRAPHS", "1"),
    # All-gather leg of the fused row-parallel path through an NVLink multicast mapping (one multimem.st, replicated
    # by the switch) when torch's symmetric memory can provide one.  0 = one peer store per rank, 1 = multicast at 4
    # ranks and more (at 2 ranks it saves no bytes and measured 10 % slower), 2 = multicast at any world size.
    "B200_USE_MULTIMEM": _int("B200_USE_MULTIMEM", 1),
    # Steps of at most this many tokens take the in-switch all-reduce + norm kernel (multimem.ld_reduce) after a plain
    # local GEMM; larger steps take the scatter GEMM + reduce / gather kernels.  0 = never.
    "B200_NVLS_AR_MAX_TOKENS": _int("B200_NVLS_AR_MAX_TOKENS", 1024),
    # Iteration budget of device-side waits on peer flags before giving up.
    "B200_PEER_WAIT_ITERS": _int("B200_PEER_WAIT_ITERS", 20_000_000),
    "B200_PP_DISABLE_ALLGATHER": _flag("B200_PP_DISABLE_ALLGATHER", "0"),
    # Peer-store all-reduce kernel for tensor-parallel reductions up to B200_CUSTOM_ALLREDUCE_MAX_BYTES
    # (larger messages stay on NCCL).
    "B200_CUSTOM_ALLREDUCE": _flag("B200_CUSTOM_ALLREDUCE", "1"),
    "B200_CUSTOM_ALLREDUCE_MAX_BYTES": _int("B200_CUSTOM_ALLREDUCE_MAX_BYTES", 8 << 20),
    # NVTX range around every forward pass (Nsight Systems / Compute timelines).
    "B200_NVTX": _flag("B200_NVTX", "0"),
    # ---- debug -------------------------------------------------------------
    "B200_FORCE_REFERENCE_OPS": _flag("B200_FORCE_REFERENCE_OPS", "0"),
    "B200_PRECISION_DUMP_DIR": _str("B200_PRECISION_DUMP_DIR", None),
    "B200_LOG_LEVEL": _str("B200_LOG_LEVEL", "INFO"),
}

_overrides: dict[str, tuple[Any, str]] = {}


def override_env(name: str, value: Any, reason: str, *, forward_to_vllm: bool = False) -> None:
    """Force ``name`` to ``value`` for this process and record why.

    The value is written to ``os.environ`` (so child processes inherit it) and
    the resolver is replaced.  With ``forward_to_vllm`` the same is done to
    ``vllm.envs.environment_variables`` if vLLM is importable.
    """
    sval = "1" if value is True else "0" if value is False else str(value)
    old = os.environ.get(name)
    os.environ[name] = sval
    environment_variables[name] = (lambda v=value: v)
    _overrides[name] = (value, reason)
    logger.info("env override %s: %r -> %r (%s)", name, old, sval, reason)
    if forward_to_vllm:
        try:
            import vllm.envs as venvs  # type: ignore

            if hasattr(venvs, "environment_variables"):
                venvs.environment_variables[name] = (lambda v=value: v)
        except Exception:  # pragma: no cover - vLLM optional
            pass


def overrides() -> dict[str, tuple[Any, str]]:
    return dict(_overrides)


def __getattr__(name: str) -> Any:
    if name in environment_variables:
        return environment_variables[name]()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return list(environment_variables.keys())
