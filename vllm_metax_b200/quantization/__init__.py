"""Quantisation registry: maps a checkpoint's ``quantization_config`` to per-layer methods.

``get_linear_method(cfg, prefix)`` returns the ``LinearMethodBase`` for the linear layer
at ``prefix`` (``None`` = unquantised bf16 tcgen05 GEMM).  Names follow the reference's
supported list (vllm_metax/platform.py:177-189): awq, gptq, compressed-tensors, fp8,
moe_wna16 (+ w8a8 int8 through compressed-tensors), mxfp4 / nvfp4 (weight-only, expanded at load).
"""
from __future__ import annotations

from typing import Callable, Optional

_REGISTRY: dict[str, Callable] = {}


def register_quantization_config(name: str):
    def deco(fn):
        _REGISTRY[name] = fn
        return fn
    return deco


def supported_quantization() -> list[str]:
    _ensure_loaded()
    return sorted(_REGISTRY)


_loaded = False


def _ensure_loaded():
    global _loaded
    if _loaded:
        return
    _loaded = True
    import importlib

    for mod in ("fp8", "int8", "wna16", "fp4"):
        try:
            importlib.import_module(f"{__name__}.{mod}")
        except ModuleNotFoundError:
            pass


def get_quant_config(cfg):
    if not cfg.quantization:
        return None
    _ensure_loaded()
    name = cfg.quantization.replace("-", "_")
    if name not in _REGISTRY:
        raise ValueError(f"unsupported quantization {cfg.quantization!r}; supported: {supported_quantization()}")
    qc = getattr(cfg, "_quant_config_obj", None)
    if qc is None:
        qc = _REGISTRY[name](cfg.quant_config)
        cfg._quant_config_obj = qc
    return qc


def get_linear_method(cfg, prefix: str):
    qc = get_quant_config(cfg)
    return None if qc is None else qc.get_linear_method(prefix)


def get_moe_method(cfg, prefix: str):
    qc = get_quant_config(cfg)
    return None if qc is None else qc.get_moe_method(prefix)
