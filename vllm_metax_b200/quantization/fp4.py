"""4-bit floating-point weight checkpoints: MXFP4 (e2m1 values, one power-of-two UE8M0 scale per 32) and NVFP4 (e2m1
values, one e4m3 scale per 16 plus a per-tensor fp32 scale).

Weight-only: the packed tensors are expanded to the model dtype once, after loading, and the layers then run the
ordinary bf16 tcgen05 GEMMs (dense) / grouped GEMMs (experts) - the checkpoint format is supported, the 4x smaller
footprint is not kept.  Two values share a byte, low nibble first.

Checkpoint tensors per linear: ``weight`` (or ``weight_packed``) uint8 ``[N, K/2]``, ``weight_scale`` ``[N, K/group]``
(uint8 exponents for MXFP4, e4m3 for NVFP4) and, for NVFP4, ``weight_scale_2`` (multiplied) or ``weight_global_scale``
(divided).  Experts carry the same tensors per expert projection.

Parity: the mxfp4 expert weights of the reference's DeepSeek-V4 path (vllm_metax/models/deepseek_v4/model.py:140-476,
1204-1240) and the fp4 entries of its quantisation list (vllm_metax/platform.py:177-189).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..layers.linear import LinearMethodBase
from . import register_quantization_config

E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def dequant_fp4(packed: torch.Tensor, scale: torch.Tensor, group: int, global_scale: Optional[torch.Tensor] = None,
                dtype=torch.bfloat16) -> torch.Tensor:
    """``packed uint8 [..., K/2]``, ``scale [..., K/group]`` (uint8 = UE8M0 exponent, else a float type) -> ``[..., K]``."""
    lut = torch.tensor(E2M1 + tuple(-v for v in E2M1), dtype=torch.float32, device=packed.device)
    b = packed.to(torch.int64)
    vals = torch.stack([lut[b & 0xF], lut[b >> 4]], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    if scale.dtype == torch.uint8:
        s = torch.exp2(scale.to(torch.float32) - 127.0)
    else:
        s = scale.to(torch.float32)
    K = vals.shape[-1]
    vals = (vals.reshape(*vals.shape[:-1], K // group, group) * s.unsqueeze(-1)).reshape(*vals.shape[:-1], K)
    if global_scale is not None:
        vals = vals * global_scale.to(torch.float32)
    return vals.to(dtype)


def quant_fp4_ref(w: torch.Tensor, kind: str):
    """Round-to-nearest reference quantiser (tests, and ``LLM.update_weights`` round trips): returns
    ``(packed, scale, global_scale | None)``."""
    group = 32 if kind == "mxfp4" else 16
    wf = w.float()
    g = wf.reshape(*wf.shape[:-1], wf.shape[-1] // group, group)
    amax = g.abs().amax(-1).clamp(min=1e-12)
    gs = None
    if kind == "mxfp4":
        e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
        scale = (e + 127).to(torch.uint8)
        s = torch.exp2(e)
    else:
        gs = (wf.abs().amax() / (6.0 * 448.0)).clamp(min=1e-12)
        scale = (amax / 6.0 / gs).to(torch.float8_e4m3fn)
        s = scale.float() * gs
        s = s.clamp(min=1e-30)
    lut = torch.tensor(E2M1)
    q = (g / s.unsqueeze(-1)).clamp(-6, 6)
    idx = (q.abs().unsqueeze(-1) - lut).abs().argmin(-1) + torch.where(q < 0, 8, 0)
    idx = idx.reshape(*wf.shape[:-1], wf.shape[-1] // 2, 2)
    packed = (idx[..., 0] | (idx[..., 1] << 4)).to(torch.uint8)
    return packed, scale, gs


def _scale_param(shape, kind: str):
    if kind == "mxfp4":
        p = nn.Parameter(torch.full(shape, 127, dtype=torch.uint8), requires_grad=False)
    else:
        p = nn.Parameter(torch.ones(shape, dtype=torch.float32).to(torch.float8_e4m3fn), requires_grad=False)
    return p


class Fp4LinearMethod(LinearMethodBase):
    def __init__(self, kind: str):
        self.kind, self.group = kind, 32 if kind == "mxfp4" else 16

    def create_weights(self, layer, in_features, out_features, dtype):
        assert in_features % self.group == 0
        layer.weight = nn.Parameter(torch.zeros(out_features, in_features // 2, dtype=torch.uint8), requires_grad=False)
        layer.weight_scale = _scale_param((out_features, in_features // self.group), self.kind)
        if self.kind == "nvfp4":          # per-tensor scales of fused projections: one value per output row
            for name in ("weight_scale_2", "weight_global_scale"):
                p = nn.Parameter(torch.ones(out_features, 1, dtype=torch.float32), requires_grad=False)
                p.output_dim, p.expand_scalar, p.is_scale = 0, True, True
                setattr(layer, name, p)
        layer._fp4_dtype = dtype

    def process_weights_after_loading(self, layer) -> None:
        if layer.weight.dtype != torch.uint8:
            return
        gs = None
        if self.kind == "nvfp4":
            gs = layer.weight_scale_2.data / layer.weight_global_scale.data
        w = dequant_fp4(layer.weight.data, layer.weight_scale.data, self.group, gs, layer._fp4_dtype)
        for name in ("weight_scale", "weight_scale_2", "weight_global_scale"):
            if hasattr(layer, name):
                delattr(layer, name)
        layer.weight = nn.Parameter(w, requires_grad=False)

    def apply(self, layer, x, bias=None, residual=None):
        return ops.gemm(x, layer.weight, bias, residual)


class Fp4MoEMethod:
    """Experts: packed ``w13 [E, 2I, H/2]`` (gate rows, then up rows) / ``w2 [E, H, I/2]`` expanded after loading to
    the interleaved bf16 layout of the grouped GEMM."""

    def __init__(self, kind: str):
        self.kind, self.group = kind, 32 if kind == "mxfp4" else 16

    def create_weights(self, layer, num_local, hidden, inter, dtype):
        g = self.group
        layer.w13_weight = nn.Parameter(torch.zeros(num_local, 2 * inter, hidden // 2, dtype=torch.uint8), requires_grad=False)
        layer.w2_weight = nn.Parameter(torch.zeros(num_local, hidden, inter // 2, dtype=torch.uint8), requires_grad=False)
        layer.w13_weight_scale = _scale_param((num_local, 2 * inter, hidden // g), self.kind)
        layer.w2_weight_scale = _scale_param((num_local, hidden, inter // g), self.kind)
        if self.kind == "nvfp4":
            for name, rows in (("w13", 2 * inter), ("w2", hidden)):
                for suffix in ("weight_scale_2", "weight_global_scale"):
                    setattr(layer, f"{name}_{suffix}", nn.Parameter(torch.ones(num_local, rows, 1), requires_grad=False))
        self.inter, self.dtype = inter, dtype

    def load_expert_weight(self, layer, param, loaded, e, shard):
        inter = self.inter
        if loaded.numel() == 1:
            loaded = loaded.reshape(1, 1).expand(inter if shard in ("w1", "w3") else param.shape[1], 1)
        loaded = loaded.reshape(loaded.shape[0], -1)
        if shard == "w1":
            param.data[e, :inter].copy_(loaded)
        elif shard == "w3":
            param.data[e, inter:].copy_(loaded)
        else:
            param.data[e].copy_(loaded)

    def process_weights_after_loading(self, layer) -> None:
        if layer.w13_weight.dtype != torch.uint8:
            return
        out = {}
        for name in ("w13", "w2"):
            gs = None
            if self.kind == "nvfp4":
                gs = getattr(layer, f"{name}_weight_scale_2").data / getattr(layer, f"{name}_weight_global_scale").data
            out[name] = dequant_fp4(getattr(layer, f"{name}_weight").data, getattr(layer, f"{name}_weight_scale").data,
                                    self.group, gs, self.dtype)
            for suffix in ("weight_scale", "weight_scale_2", "weight_global_scale"):
                if hasattr(layer, f"{name}_{suffix}"):
                    delattr(layer, f"{name}_{suffix}")
        I = self.inter
        w13 = torch.empty_like(out["w13"])
        w13[:, 0::2], w13[:, 1::2] = out["w13"][:, :I], out["w13"][:, I:]
        layer.w13_weight = nn.Parameter(w13, requires_grad=False)
        layer.w2_weight = nn.Parameter(out["w2"], requires_grad=False)

    def apply(self, layer, x, topk_weights, topk_ids, shared_out=None):
        from ..layers.fused_moe import fused_experts

        return fused_experts(x, layer.w13_weight, layer.w2_weight, topk_weights, topk_ids, layer.num_local,
                             layer.expert_map, shared_out)


class Fp4Config:
    def __init__(self, cfg: dict, kind: str):
        self.kind = kind
        self.ignored = list(cfg.get("ignored_layers") or cfg.get("ignore") or cfg.get("exclude_modules")
                            or cfg.get("modules_to_not_convert") or [])

    def _skip(self, prefix: str) -> bool:
        return (any(ig.strip("*") in prefix for ig in self.ignored) or prefix.endswith("lm_head")
                or prefix.endswith(".gate") or prefix.endswith("shared_expert_gate"))

    def get_linear_method(self, prefix: str):
        return None if self._skip(prefix) else Fp4LinearMethod(self.kind)

    def get_moe_method(self, prefix: str):
        return Fp4MoEMethod(self.kind)


@register_quantization_config("mxfp4")
def _mxfp4(cfg: dict):
    return Fp4Config(cfg, "mxfp4")


@register_quantization_config("nvfp4")
def _nvfp4(cfg: dict):
    return Fp4Config(cfg, "nvfp4")


@register_quantization_config("modelopt_fp4")
def _modelopt_fp4(cfg: dict):
    return Fp4Config(cfg, "nvfp4")


@register_quantization_config("modelopt")
def _modelopt(cfg: dict):
    algo = str(cfg.get("quant_algo", (cfg.get("quantization") or {}).get("quant_algo", ""))).upper()
    if "FP4" not in algo:
        raise ValueError(f"modelopt quant_algo {algo!r} is not supported (NVFP4 is)")
    return Fp4Config(cfg, "nvfp4")
