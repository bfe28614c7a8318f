"""Out-of-tree implementations of vLLM ``CustomOp`` layers on this package's kernels.

One table drives the registration: (upstream module, class name, forward_oot).  Each entry becomes a
subclass of the upstream layer whose ``forward_oot`` calls ``vllm_metax_b200._custom_ops``; vLLM picks it
up through ``CustomOp.register_oot`` when the platform is out-of-tree.
Parity: vllm_metax/registry/custom_ops/activation.py:17-73 (ten activations), layernorm.py:6-20
(RMSNorm, GemmaRMSNorm, RMSNormGated), layers/rotary_embedding, layers/minimax_rms_norm.
"""
from __future__ import annotations

import importlib
from typing import Callable, Optional

import torch

from .. import _custom_ops as ops

REGISTERED: dict[str, type] = {}


def _gated(name: str, **fixed) -> Callable:
    def fwd(self, x: torch.Tensor) -> torch.Tensor:
        p0 = p1 = 0.0
        if name == "fatrelu":
            p0 = float(getattr(self, "threshold", 0.0))
        if name == "swigluoai":
            p0, p1 = float(getattr(self, "alpha", 1.702)), float(getattr(self, "limit", 7.0))
        if name in ("swiglustep", "silu_clamp"):
            p1 = float(getattr(self, "limit", getattr(self, "swiglu_limit", 7.0)))
        return ops.act_and_mul(x, name if name != "silu_clamp" else "swiglustep", p0=p0, p1=p1)

    return fwd


def _plain(name: str) -> Callable:
    def fwd(self, x: torch.Tensor) -> torch.Tensor:
        return ops.activation(x, name)

    return fwd


def _rms_norm(gemma: bool) -> Callable:
    def fwd(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        eps = float(getattr(self, "variance_epsilon", getattr(self, "eps", 1e-6)))
        w = self.weight.data if getattr(self, "has_weight", True) else torch.ones(x.shape[-1], dtype=x.dtype, device=x.device)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if residual is not None:
            r2 = residual.reshape(-1, shape[-1])
            ops.fused_add_rms_norm(x2, r2, w, eps, gemma=gemma)
            return x2.reshape(shape), r2.reshape(shape)
        return ops.rms_norm(x2, w, eps, gemma=gemma).reshape(shape)

    return fwd


def _rms_norm_gated(self, x: torch.Tensor, z: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x) * silu(z) (norm_before_gate) as used by Mamba-2 / gated delta-net blocks."""
    eps = float(getattr(self, "eps", 1e-6))
    if z is not None and not getattr(self, "norm_before_gate", True):
        x = x * torch.nn.functional.silu(z.float()).to(x.dtype)
        z = None
    y = ops.rms_norm(x.reshape(-1, x.shape[-1]), self.weight.data, eps).reshape(x.shape)
    if z is not None:
        y = y * torch.nn.functional.silu(z.float()).to(y.dtype)
    return y


_TABLE = [
    ("vllm.model_executor.layers.activation", "SiluAndMul", _gated("silu")),
    ("vllm.model_executor.layers.activation", "MulAndSilu", _gated("mul_silu")),
    ("vllm.model_executor.layers.activation", "GeluAndMul", None),           # approximate flag read at call
    ("vllm.model_executor.layers.activation", "FatreluAndMul", _gated("fatrelu")),
    ("vllm.model_executor.layers.activation", "SwigluOAIAndMul", _gated("swigluoai")),
    ("vllm.model_executor.layers.activation", "SwigluStepAndMul", _gated("swiglustep")),
    ("vllm.model_executor.layers.activation", "SiluAndMulWithClamp", _gated("silu_clamp")),
    ("vllm.model_executor.layers.activation", "NewGELU", _plain("gelu_new")),
    ("vllm.model_executor.layers.activation", "FastGELU", _plain("gelu_fast")),
    ("vllm.model_executor.layers.activation", "QuickGELU", _plain("gelu_quick")),
    ("vllm.model_executor.layers.layernorm", "RMSNorm", _rms_norm(False)),
    ("vllm.model_executor.layers.layernorm", "GemmaRMSNorm", _rms_norm(True)),
    ("vllm.model_executor.layers.layernorm", "RMSNormGated", _rms_norm_gated),
]


def _gelu_and_mul(self, x: torch.Tensor) -> torch.Tensor:
    return ops.act_and_mul(x, "gelu_tanh" if getattr(self, "approximate", "none") == "tanh" else "gelu")


def register_all() -> dict[str, type]:
    for mod_name, cls_name, fwd in _TABLE:
        try:
            base = getattr(importlib.import_module(mod_name), cls_name)
        except (ImportError, AttributeError):
            continue
        if cls_name in REGISTERED or not hasattr(base, "register_oot"):
            continue
        impl = fwd if fwd is not None else _gelu_and_mul
        sub = type(f"B200{cls_name}", (base,), {"forward_oot": impl, "__doc__": f"{cls_name} on sm_100a kernels"})
        try:
            base.register_oot(sub)
        except AssertionError:      # another plugin registered this layer first
            continue
        REGISTERED[cls_name] = sub
    return REGISTERED


register_all()
