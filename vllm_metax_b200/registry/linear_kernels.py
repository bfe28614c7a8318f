"""Linear kernels offered to vLLM's kernel selection for the out-of-tree platform.

* ``B200Fp8BlockScaledMMKernel``  block-scaled fp8 (1x128 activations, 128x128 weights) -> tcgen05 kind::f8f6f4
* ``B200Int8ScaledMMKernel``      W8A8 int8, static or dynamic per-token activations, optional zero point
                                  -> tcgen05 kind::i8 with scales / azp / bias in the epilogue
* ``B200WNA16LinearKernel``       4/8-bit weight-only (GPTQ / AWQ / compressed-tensors) incl. act-order
                                  -> fused dequantise + tcgen05 kind::f16, repacked once at load
Parity: vllm_metax/registry/linear_kernels/fp8.py:29-49, int8.py:33-79, mp.py:22-218.
"""
from __future__ import annotations

import torch

from .. import _custom_ops as ops
from ..quantization import wna16 as W

try:
    from vllm.model_executor.kernels.linear import register_linear_kernel
    from vllm.model_executor.kernels.linear.mixed_precision.MPLinearKernel import MPLinearKernel, MPLinearLayerConfig
    from vllm.model_executor.kernels.linear.scaled_mm.BlockScaledMMLinearKernel import Fp8BlockScaledMMLinearKernel
    from vllm.model_executor.kernels.linear.scaled_mm.ScaledMMLinearKernel import (Int8ScaledMMLinearKernel,
                                                                                  Int8ScaledMMLinearLayerConfig)
    from vllm.platforms import PlatformEnum

    _OK = True
except Exception:  # pragma: no cover - vLLM layout differs
    _OK = False
    MPLinearKernel = Fp8BlockScaledMMLinearKernel = Int8ScaledMMLinearKernel = object  # type: ignore


class B200Fp8BlockScaledMMKernel(Fp8BlockScaledMMLinearKernel):
    @classmethod
    def is_supported(cls, compute_capability=None):
        return True, None

    @classmethod
    def can_implement(cls, config):
        return True, None

    def apply_block_scaled_mm(self, A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor) -> torch.Tensor:
        return ops.fp8_block_scaled_mm(A, As, B, Bs, self.config.out_dtype)


class B200Int8ScaledMMKernel(Int8ScaledMMLinearKernel):
    @classmethod
    def is_supported(cls, compute_capability=None):
        return True, None

    @classmethod
    def can_implement(cls, c):
        return True, None

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        w_q, w_s, i_s, i_zp, azp_adj = self.layer_param_names
        w = getattr(layer, w_q).data
        if w.shape[0] != getattr(layer, w_s).data.shape[0] and w.shape[1] == getattr(layer, w_s).data.numel():
            w = w.t()
        setattr(layer, w_q, torch.nn.Parameter(w.contiguous(), requires_grad=False))      # [N, K]
        setattr(layer, w_s, torch.nn.Parameter(getattr(layer, w_s).data.float().reshape(-1).contiguous(), requires_grad=False))
        if not self.config.input_symmetric:
            adj = getattr(layer, w_q).data.to(torch.int32).sum(dim=1, dtype=torch.int32)
            zp = getattr(layer, i_zp, None)
            if self.config.is_static_input_scheme and zp is not None:
                adj = adj * zp.data.to(torch.int32)
            setattr(layer, azp_adj, torch.nn.Parameter(adj.contiguous(), requires_grad=False))

    def apply_weights(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        w, ws, i_s, i_zp, adj = self._get_layer_params(layer)
        sym = self.config.input_symmetric
        x2 = x.reshape(-1, x.shape[-1])
        if self.config.is_static_input_scheme:
            xq, xs, _ = ops.scaled_int8_quant(x2, scale=i_s, azp=None if sym else i_zp, symmetric=sym)
            azp = None
        else:
            xq, xs, azp = ops.scaled_int8_quant(x2, symmetric=sym)
        y = ops.scaled_mm(xq, w, xs, ws, x.dtype, azp=azp, azp_adj=None if sym else adj, bias=bias)
        return y.reshape(*x.shape[:-1], -1)


class B200WNA16LinearKernel(MPLinearKernel):
    """Expects GPTQ-style parameters: ``w_q`` int32 packed along K ``[K/pack, N]``, ``w_s [K/g, N]``,
    optional ``w_zp`` int32 packed along N ``[K/g, N/pack]`` and ``g_idx``."""

    @classmethod
    def get_min_capability(cls) -> int:
        return 100

    @classmethod
    def can_implement(cls, c):
        bits = getattr(c.weight_type, "size_bits", 4)
        if bits not in (4, 8):
            return False, "only 4- and 8-bit weights"
        k = c.partition_weight_shape[0]
        g = k if c.group_size in (-1, None) else c.group_size
        if k % 64 or g % 32 or k % g:
            return False, "K must be a multiple of 64 and of the group size (itself a multiple of 32)"
        return True, None

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        c = self.config
        bits = c.weight_type.size_bits
        w_q, w_s, w_zp, w_gidx = self._get_weight_params(layer)
        k = c.partition_weight_shape[0]
        group = k if c.group_size in (-1, None) else c.group_size
        q_nk = W.unpack_int32(w_q.data, bits, 0).t().contiguous()
        z = None
        if c.zero_points and w_zp is not None:
            z = W.unpack_int32(w_zp.data, bits, 1).to(torch.int32)
        elif getattr(c.weight_type, "bias", 0):
            z = None      # symmetric types carry bias 2^(bits-1): the default zero point
        perm = None
        if c.has_g_idx and w_gidx is not None and w_gidx.numel() == k:
            g_idx = w_gidx.data.long()
            if not torch.equal(g_idx, torch.arange(k, device=g_idx.device) // group):
                perm = torch.argsort(g_idx, stable=True)
                q_nk = q_nk[:, perm]
        qc, s, zc = W.canonical_from_values(q_nk, w_s.data, z, bits, c.act_type)
        layer.b200_q = torch.nn.Parameter(qc, requires_grad=False)
        layer.b200_s = torch.nn.Parameter(s, requires_grad=False)
        layer.b200_z = torch.nn.Parameter(zc, requires_grad=False)
        layer.b200_perm, layer.b200_bits, layer.b200_group = perm, bits, group
        self._transform_param(layer, self.w_q_name, lambda p: torch.empty(0, dtype=p.dtype, device=p.device))

    def apply_weights(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        if layer.b200_perm is not None:
            x2 = x2.index_select(-1, layer.b200_perm)
        y = ops.wna16_gemm(x2, layer.b200_q, layer.b200_s, layer.b200_z, layer.b200_bits, layer.b200_group, bias=bias)
        return y.reshape(*x.shape[:-1], -1)


if _OK:
    register_linear_kernel(B200Int8ScaledMMKernel, PlatformEnum.OOT, "int8")
    register_linear_kernel(B200WNA16LinearKernel, PlatformEnum.OOT, "mp")
