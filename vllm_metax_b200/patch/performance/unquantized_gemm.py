"""Unquantised linear layers of upstream vLLM on this package's tcgen05 GEMMs.

Upstream's ``UnquantizedLinearMethod.apply`` calls the function ``dispatch_unquantized_gemm()`` returned when the
layer was built; on a CUDA-like out-of-tree platform that is ``default_unquantized_gemm`` =
``torch.nn.functional.linear`` (vllm/model_executor/layers/utils.py:92-98, 321-327).  The replacement sends 16-bit
2-D problems to ``ops.gemm`` (CTA-pair / tile / split-K / stream-K kernels picked by shape) and leaves everything
else (fp32, odd strides) on the library call.
Parity: the reference reaches its vendor GEMM through the same hook (vllm_metax/patch/... utils dispatch).
"""
from __future__ import annotations

import torch

from ... import _custom_ops as ops
from ..utils import patch


@patch("vllm.model_executor.layers.utils", "default_unquantized_gemm")
def default_unquantized_gemm(layer, x, weight, bias=None):
    if (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and weight.dim() == 2
            and weight.stride(1) == 1 and weight.shape[1] % 8 == 0 and weight.stride(0) % 8 == 0
            and weight.shape[0] % 8 == 0):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.shape[0] > 0:
            y = ops.gemm(x2, weight, bias)
            return y.view(*x.shape[:-1], weight.shape[0])
    return torch.nn.functional.linear(x, weight, bias)
