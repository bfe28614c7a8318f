"""Block-scaled fp8 (DeepSeek-V3 style) checkpoints.

Weights are e4m3 with one f32 ``weight_scale_inv`` per 128 x 128 block; activations are
quantised dynamically 1 x 128 per token before every GEMM.  Linear layers and MoE experts both
run on the tcgen05 block-scaled GEMM (``csrc/gemm_fp8_blockscale.cu``).

Parity: vllm_metax/registry/quant_config/fp8.py:47-170 (MacaFp8Config, Fp8MoEMethod,
weight_block_size [128, 128], dynamic activation scheme),
registry/linear_kernels/fp8.py:29-49 (MctlassFp8BlockScaledMMKernel).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..layers.linear import LinearMethodBase
from . import register_quantization_config

BLOCK = 128


def _scale_param(*shape) -> nn.Parameter:
    p = nn.Parameter(torch.ones(*shape, dtype=torch.float32), requires_grad=False)
    p.is_scale = True
    return p


class Fp8BlockLinearMethod(LinearMethodBase):
    def create_weights(self, layer, in_features, out_features, dtype):
        layer.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.float8_e4m3fn),
                                    requires_grad=False)
        layer.weight_scale_inv = _scale_param((out_features + BLOCK - 1) // BLOCK, (in_features + BLOCK - 1) // BLOCK)
        # block-scale tensors follow the sharding of the weight at 1/128 granularity
        layer.weight_scale_inv.block_n = BLOCK
        layer.weight_scale_inv.output_dim = 0
        layer.weight_scale_inv.input_dim = 1

    def apply(self, layer, x, bias=None, residual=None):
        xq, xs = ops.per_token_group_quant_fp8(x, BLOCK)
        y = ops.fp8_block_scaled_mm(xq, xs, layer.weight, layer.weight_scale_inv, x.dtype)
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        return y


class Fp8MoEMethod:
    """Experts with block-scaled fp8 weights: w13 [E, 2I, H] (gate rows then up rows), w2 [E, H, I]."""

    def create_weights(self, layer, num_local, hidden, inter, dtype):
        layer.w13_weight = nn.Parameter(torch.empty(num_local, 2 * inter, hidden, dtype=torch.float8_e4m3fn),
                                        requires_grad=False)
        layer.w2_weight = nn.Parameter(torch.empty(num_local, hidden, inter, dtype=torch.float8_e4m3fn),
                                       requires_grad=False)
        layer.w13_weight_scale_inv = _scale_param(num_local, (2 * inter + BLOCK - 1) // BLOCK, (hidden + BLOCK - 1) // BLOCK)
        layer.w2_weight_scale_inv = _scale_param(num_local, (hidden + BLOCK - 1) // BLOCK, (inter + BLOCK - 1) // BLOCK)
        self.inter = inter
        self.dtype = dtype

    def load_expert_weight(self, layer, param, loaded, e, shard):
        is_scale = param.dtype == torch.float32
        unit = BLOCK if is_scale else 1
        inter = self.inter
        if shard == "w1":
            param.data[e, : (inter + unit - 1) // unit].copy_(loaded)
        elif shard == "w3":
            off = inter // unit
            param.data[e, off: off + loaded.shape[0]].copy_(loaded)
        else:
            param.data[e].copy_(loaded)

    def apply(self, layer, x, topk_weights, topk_ids, shared_out=None):
        T = x.shape[0]
        topk = topk_ids.shape[1]
        sorted_ids, block_expert, total, inv = ops.moe_align_block_size(topk_ids, 128, layer.num_local,
                                                                        layer.expert_map, want_inverse=True)
        a = ops.moe_gather(x, sorted_ids, total, topk)
        aq, a_s = ops.per_token_group_quant_fp8(a, BLOCK)
        h = ops.fp8_block_scaled_mm(aq, a_s, layer.w13_weight, layer.w13_weight_scale_inv, x.dtype, block_expert, total)
        hq, h_s = ops.silu_and_mul_per_block_quant(h, BLOCK)
        y = ops.fp8_block_scaled_mm(hq, h_s, layer.w2_weight, layer.w2_weight_scale_inv, x.dtype, block_expert, total)
        return ops.moe_combine(y, topk_weights, inv, T, shared_out)


    # Sequence-parallel MoE over the NVLink dispatch / combine kernels: tokens travel as e4m3 rows with one scale per
    # 128 channels (the dispatch kernel quantises them), so the rows this rank receives feed the first grouped GEMM
    # without another quantisation pass.
    a2a_wire_fp8 = True

    def apply_sorted(self, layer, a, a_scale, block_expert, total):
        """Expert MLPs on expert-sorted rows that arrive quantised: ``a [padded, H]`` e4m3 bytes, ``a_scale
        [padded, H / 128]``.  Mirrors the reference's masked / batched expert path behind its low-latency dispatch
        (model_executor/layers/fused_moe/experts/batched_deep_gemm_moe.py:248-329)."""
        dt = self.dtype
        aq = a.view(torch.float8_e4m3fn) if a.dtype == torch.uint8 else a
        h = ops.fp8_block_scaled_mm(aq, a_scale, layer.w13_weight, layer.w13_weight_scale_inv, dt, block_expert, total)
        hq, h_s = ops.silu_and_mul_per_block_quant(h, BLOCK)
        return ops.fp8_block_scaled_mm(hq, h_s, layer.w2_weight, layer.w2_weight_scale_inv, dt, block_expert, total)


class Fp8Config:
    """``quantization_config`` of an fp8 checkpoint: ``{"quant_method": "fp8", "weight_block_size": [128, 128],
    "activation_scheme": "dynamic"}``.  Layers listed in ``ignored_layers`` / not matching stay bf16."""

    def __init__(self, cfg: dict):
        self.block = tuple(cfg.get("weight_block_size") or (BLOCK, BLOCK))
        if self.block != (BLOCK, BLOCK):
            raise ValueError("only 128x128 weight blocks are supported")
        if cfg.get("activation_scheme", "dynamic") != "dynamic":
            raise ValueError("only dynamic activation quantisation is supported")
        self.ignored = list(cfg.get("ignored_layers") or cfg.get("modules_to_not_convert") or [])

    def _skip(self, prefix: str) -> bool:
        return any(ig in prefix for ig in self.ignored) or prefix.endswith("lm_head") or ".gate" == prefix[-5:]

    def get_linear_method(self, prefix: str) -> Optional[LinearMethodBase]:
        return None if self._skip(prefix) else Fp8BlockLinearMethod()

    def get_moe_method(self, prefix: str):
        return Fp8MoEMethod()


@register_quantization_config("fp8")
def _make(cfg: dict) -> Fp8Config:
    return Fp8Config(cfg)
