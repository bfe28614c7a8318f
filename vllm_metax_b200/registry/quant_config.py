"""Quantisation names the out-of-tree platform accepts, and how vLLM's configs reach this package's kernels.

vLLM keeps its own ``QuantizationConfig`` classes (weight creation / loading stay upstream); they select a
linear kernel through the kernel registry, where ``registry/linear_kernels.py`` supplies the tcgen05
implementations for the out-of-tree platform.  What remains here: AWQ checkpoints are converted to the
GPTQ packing on load so that ONE weight-only kernel serves both (``AwqToGptqMixin``), and the list of
supported method names.
Parity: vllm_metax/registry/quant_config/auto_awq.py:30-173 (AWQ -> GPTQ repack at load), auto_gptq.py:17-46,
compressed_tensors.py:43-105, fp8.py:47-170, moe_wna16.py:29-92.
"""
from __future__ import annotations

import torch

from ..quantization import wna16 as W

SUPPORTED = ["awq", "auto_awq", "gptq", "auto_gptq", "compressed-tensors", "moe_wna16", "fp8", "gguf"]


def awq_to_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, bits: int = 4):
    """AWQ tensors (``[K, N/8]`` / ``[K/g, N/8]``, AWQ nibble order) -> GPTQ v2 tensors
    (``qweight [K/8, N]`` packed along K, ``qzeros [K/g, N/8]`` sequential order, zero point stored as is)."""
    q_nk, z = W.awq_to_values(qweight, qzeros, bits)
    return W.pack_int32(q_nk.t().contiguous(), bits, 0), W.pack_int32(z, bits, 1)


class AwqToGptqMixin:
    """Mix into an AWQ linear method: repack once after loading, then behave like GPTQ (no act-order)."""

    def repack(self, layer: torch.nn.Module) -> None:
        qw, qz = awq_to_gptq(layer.qweight.data, layer.qzeros.data)
        layer.qweight = torch.nn.Parameter(qw, requires_grad=False)
        layer.qzeros = torch.nn.Parameter(qz, requires_grad=False)


def _register() -> None:
    try:
        from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, register_quantization_config
        from vllm.model_executor.layers.quantization.awq import AWQConfig, AWQLinearMethod
    except Exception:
        return
    if "auto_awq" in QUANTIZATION_METHODS:
        return

    class B200AWQLinearMethod(AWQLinearMethod, AwqToGptqMixin):
        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            q_nk, z = W.awq_to_values(layer.qweight.data, layer.qzeros.data, 4)
            qc, s, zc = W.canonical_from_values(q_nk, layer.scales.data, z, 4, layer.scales.dtype)
            layer.b200_q = torch.nn.Parameter(qc, requires_grad=False)
            layer.b200_s = torch.nn.Parameter(s, requires_grad=False)
            layer.b200_z = torch.nn.Parameter(zc, requires_grad=False)
            layer.qweight = torch.nn.Parameter(torch.empty(0, dtype=torch.int32, device=qc.device), requires_grad=False)

        def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias=None) -> torch.Tensor:
            from .. import _custom_ops as ops

            x2 = x.reshape(-1, x.shape[-1])
            y = ops.wna16_gemm(x2, layer.b200_q, layer.b200_s, layer.b200_z, 4, self.quant_config.group_size, bias=bias)
            return y.reshape(*x.shape[:-1], -1)

    @register_quantization_config("auto_awq")
    class B200AWQConfig(AWQConfig):
        @classmethod
        def get_name(cls):
            return "auto_awq"

        def get_quant_method(self, layer, prefix: str):
            m = super().get_quant_method(layer, prefix)
            return B200AWQLinearMethod(self) if isinstance(m, AWQLinearMethod) else m


_register()
