"""W8A8 int8 checkpoints (compressed-tensors ``int-quantized`` and the plain ``w8a8_int8`` layout).

Weights are int8 ``[N, K]`` with per-channel (or per-tensor) f32 scales; activations are quantised per
token on the fly (symmetric, or asymmetric with a zero point) or with a static per-tensor scale.  The
GEMM runs on tcgen05 ``kind::i8`` with scales, zero-point correction and bias in its epilogue
(``csrc/gemm_scaled_mm.cu``); experts use the grouped mode of the same kernel.

Parity: vllm_metax/registry/linear_kernels/int8.py:33-79 (MctlassScaledMMLinearKernel: scaled_int8_quant
+ scaled-mm with azp), registry/quant_config/compressed_tensors_moe/compressed_tensors_w8a8_int8.py:43-134,
patch/bugfix/int8_w8a8/load_weight.py:19-88 (fused w13 scale loading).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..layers.linear import LinearMethodBase
from . import register_quantization_config


def _f32(*shape, fill=1.0):
    p = nn.Parameter(torch.full(shape, fill, dtype=torch.float32), requires_grad=False)
    p.is_scale = True
    return p


class Int8LinearMethod(LinearMethodBase):
    def __init__(self, static_act: bool = False, act_sym: bool = True, per_channel: bool = True):
        self.static_act, self.act_sym, self.per_channel = static_act, act_sym, per_channel

    def create_weights(self, layer, in_features, out_features, dtype):
        layer.weight = nn.Parameter(torch.zeros(out_features, in_features, dtype=torch.int8), requires_grad=False)
        # per-tensor scales of fused projections are expanded to per channel so shards keep their own value
        layer.weight_scale = _f32(out_features, 1)
        layer.weight_scale.output_dim = 0
        layer.weight_scale.expand_scalar = True
        if self.static_act:
            layer.input_scale = _f32(1)
            if not self.act_sym:
                layer.input_zero_point = nn.Parameter(torch.zeros(1, dtype=torch.int32), requires_grad=False)
        layer.azp_adj = None

    def process_weights_after_loading(self, layer) -> None:
        if not self.act_sym and layer.azp_adj is None:
            adj = layer.weight.data.to(torch.int32).sum(dim=1, dtype=torch.int32)
            if self.static_act:   # per-tensor zero point: fold it into the correction once
                adj = adj * layer.input_zero_point.data.to(torch.int32)
            layer.azp_adj = adj.contiguous()

    def apply(self, layer, x, bias=None, residual=None):
        azp = None
        if self.static_act:
            zp = None if self.act_sym else layer.input_zero_point
            xq, xs, _ = ops.scaled_int8_quant(x, scale=layer.input_scale, azp=zp, symmetric=self.act_sym)
        else:
            xq, xs, azp = ops.scaled_int8_quant(x, symmetric=self.act_sym)
        y = ops.scaled_mm(xq, layer.weight, xs, layer.weight_scale, x.dtype, azp=azp,
                          azp_adj=None if self.act_sym else layer.azp_adj, bias=bias)
        if residual is not None:
            y = y + residual
        return y


class Int8MoEMethod:
    """Experts W8A8: ``w13 [E, 2I, H]`` int8 (gate rows, then up rows), ``w2 [E, H, I]``, per-channel scales.
    Activations are quantised per token before each grouped GEMM."""

    def create_weights(self, layer, num_local, hidden, inter, dtype):
        layer.w13_weight = nn.Parameter(torch.zeros(num_local, 2 * inter, hidden, dtype=torch.int8), requires_grad=False)
        layer.w2_weight = nn.Parameter(torch.zeros(num_local, hidden, inter, dtype=torch.int8), requires_grad=False)
        layer.w13_weight_scale = _f32(num_local, 2 * inter, 1)
        layer.w2_weight_scale = _f32(num_local, hidden, 1)
        self.inter, self.dtype = inter, dtype

    def load_expert_weight(self, layer, param, loaded, e, shard):
        inter = self.inter
        if param.dtype == torch.float32 and loaded.numel() == 1:      # per-tensor scale -> every channel of the shard
            loaded = loaded.reshape(1, 1).expand(inter if shard in ("w1", "w3") else param.shape[1], 1)
        loaded = loaded.reshape(loaded.shape[0], -1)
        if shard == "w1":
            param.data[e, :inter].copy_(loaded)
        elif shard == "w3":
            param.data[e, inter:].copy_(loaded)
        else:
            param.data[e].copy_(loaded)

    def apply(self, layer, x, topk_weights, topk_ids, shared_out=None):
        T, topk = x.shape[0], topk_ids.shape[1]
        sorted_ids, block_expert, total, inv = ops.moe_align_block_size(topk_ids, 128, layer.num_local,
                                                                        layer.expert_map, want_inverse=True)
        a = ops.moe_gather(x, sorted_ids, total, topk)
        aq, a_s, _ = ops.scaled_int8_quant(a)
        h = ops.scaled_mm(aq, layer.w13_weight, a_s, layer.w13_weight_scale, x.dtype, block_expert=block_expert,
                          total_padded=total)
        h = ops.silu_and_mul(h)
        hq, h_s, _ = ops.scaled_int8_quant(h)
        y = ops.scaled_mm(hq, layer.w2_weight, h_s, layer.w2_weight_scale, x.dtype, block_expert=block_expert,
                          total_padded=total)
        return ops.moe_combine(y, topk_weights, inv, T, shared_out)


class W4A8Int8MoEMethod(Int8MoEMethod):
    """Experts with 4-bit channel-wise weights and dynamic per-token int8 activations (compressed-tensors
    ``pack-quantized`` weights + 8-bit ``input_activations``): the nibbles are expanded to int8 values in [-8, 7] as
    they are loaded and the layer then IS a W8A8 layer - int8 activations x int8 weights on the ``kind::i8`` tensor
    cores, per-token x per-channel scales in the epilogue.  Weights take one byte per value in memory (twice the
    checkpoint), which buys the integer tensor-core rate; group-wise 4-bit weights stay on the weight-only kernel
    (``WNA16MoEMethod``), whose group scales the W8A8 epilogue cannot apply.
    Parity: vllm_metax/registry/quant_config/compressed_tensors_moe/compressed_tensors_moe_w4a8_int4.py:33-459."""

    def __init__(self, bits: int = 4):
        self.bits = bits
        self._staging: dict = {}

    def load_expert_tensor(self, layer, e: int, shard: str, kind: str, tensor: torch.Tensor) -> None:
        if kind not in ("weight_packed", "weight_scale"):
            return                                        # weight_shape and friends carry nothing the layer needs
        st = self._staging.setdefault((e, shard), {})
        st[kind] = tensor
        if len(st) < 2:
            return
        del self._staging[(e, shard)]
        from .wna16 import unpack_int32

        q = unpack_int32(st["weight_packed"], self.bits, 1).to(torch.int16) - (1 << (self.bits - 1))   # [N, K] signed
        scale = st["weight_scale"].float().reshape(q.shape[0], -1)
        if scale.shape[1] != 1:
            raise ValueError("W4A8 with int8 activations needs channel-wise weight scales (one per output row)")
        w, s_ = (layer.w2_weight, layer.w2_weight_scale) if shard == "w2" else (layer.w13_weight, layer.w13_weight_scale)
        self.load_expert_weight(layer, w, q.to(torch.int8), e, shard)
        self.load_expert_weight(layer, s_, scale, e, shard)


class Int8Config:
    """``{"quant_method": "w8a8_int8", "activation_scheme": "dynamic" | "static", "symmetric": true}``."""

    def __init__(self, cfg: dict):
        self.static_act = cfg.get("activation_scheme", "dynamic") == "static"
        self.act_sym = bool(cfg.get("symmetric", True))
        self.ignored = list(cfg.get("ignored_layers") or cfg.get("ignore") or [])

    def _skip(self, prefix: str) -> bool:
        return any(ig in prefix for ig in self.ignored) or prefix.endswith("lm_head") or prefix.endswith(".gate")

    def get_linear_method(self, prefix: str) -> Optional[LinearMethodBase]:
        return None if self._skip(prefix) else Int8LinearMethod(self.static_act, self.act_sym)

    def get_moe_method(self, prefix: str):
        return Int8MoEMethod()


register_quantization_config("w8a8_int8")(Int8Config)
register_quantization_config("int8")(Int8Config)
