"""Weight-only quantised checkpoints (4/8-bit weights, 16-bit activations): GPTQ, AWQ,
compressed-tensors ``pack-quantized`` and ``moe_wna16``.

Every format is converted ONCE at load into the canonical layout of the tcgen05 weight-only GEMM
(``csrc/gemm_wna16_tcgen05.cu``): ``qweight uint8 [N, K*bits/8]`` K-contiguous with the nibble
interleave the dequantiser expects, ``scales [K/g, N]`` and biased ``zeros [K/g, N]`` in the activation
dtype.  Activation reordering (GPTQ ``desc_act``) becomes a K permutation of the weight plus a gather
of the activation columns.  Dense layers and MoE experts share the kernel (grouped mode for experts).

Parity: vllm_metax/registry/quant_config/auto_awq.py:30-173 (AWQ -> GPTQ-order repack at load),
auto_gptq.py:17-46, compressed_tensors.py:43-105, compressed_tensors_moe/*_wna16.py:25-78,
*_w4a8_int4.py:33-459, moe_wna16.py:29-92, registry/linear_kernels/mp.py:22-218
(MacaExllamaLinearKernel: perm / act-order handling, bf16 support).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from ..layers.linear import LinearMethodBase
from . import register_quantization_config

_AWQ_REVERSE = (0, 4, 1, 5, 2, 6, 3, 7)       # logical column j of an AWQ word sits in nibble _AWQ_REVERSE[j]
_B200_NIBBLE = (0, 2, 4, 6, 1, 3, 5, 7)       # nibble p of a canonical 32-bit word holds element _B200_NIBBLE[p]


# ----------------------------------------------------------------------------- bit packing helpers
def unpack_int32(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """int32 tensor with 32/bits values per word (little-end first) along ``dim`` -> uint8 values."""
    per = 32 // bits
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    p = packed.to(torch.int32).unsqueeze(dim + 1 if dim >= 0 else dim)
    shape = [1] * p.dim()
    shape[dim + 1 if dim >= 0 else dim] = per
    vals = (p >> shifts.view(shape)) & ((1 << bits) - 1)
    out_shape = list(packed.shape)
    out_shape[dim] *= per
    return vals.reshape(out_shape).to(torch.uint8)


def pack_int32(vals: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    per = 32 // bits
    v = vals.to(torch.int64).movedim(dim, -1)
    v = v.reshape(*v.shape[:-1], v.shape[-1] // per, per)
    shifts = torch.arange(per, device=vals.device, dtype=torch.int64) * bits
    word = (v << shifts).sum(-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return word.movedim(-1, dim)


def pack_canonical(q_nk: torch.Tensor, bits: int) -> torch.Tensor:
    """``q_nk`` uint8 values ``[..., N, K]`` -> kernel layout ``uint8 [..., N, K*bits/8]``."""
    if bits == 8:
        return q_nk.to(torch.uint8).contiguous()
    assert bits == 4 and q_nk.shape[-1] % 8 == 0
    v = q_nk.to(torch.int64).reshape(*q_nk.shape[:-1], q_nk.shape[-1] // 8, 8)
    word = torch.zeros(v.shape[:-1], dtype=torch.int64, device=q_nk.device)
    for p, e in enumerate(_B200_NIBBLE):
        word |= v[..., e] << (4 * p)
    b = torch.stack([(word >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)
    return b.reshape(*q_nk.shape[:-1], q_nk.shape[-1] // 2).contiguous()


def unpack_canonical(qc: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of ``pack_canonical`` -> uint8 values ``[..., N, K]``."""
    if bits == 8:
        return qc
    b = qc.to(torch.int64).reshape(*qc.shape[:-1], qc.shape[-1] // 4, 4)
    word = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)
    out = torch.empty(*word.shape, 8, dtype=torch.uint8, device=qc.device)
    for p, e in enumerate(_B200_NIBBLE):
        out[..., e] = ((word >> (4 * p)) & 0xF).to(torch.uint8)
    return out.reshape(*qc.shape[:-1], qc.shape[-1] * 2)


def zero_bias(bits: int, dtype: torch.dtype) -> float:
    """Offset folded into the stored zero points (see the kernel's exponent-splice dequantiser)."""
    if bits == 8:
        return 0.0
    return 1024.0 if dtype == torch.float16 else 128.0


def canonical_from_values(q_nk, scales_gn, zeros_gn, bits: int, dtype: torch.dtype):
    """``q_nk [..,N,K]`` values, ``scales_gn [..,K/g,N]``, ``zeros_gn`` integer zero points or None (symmetric)."""
    qc = pack_canonical(q_nk, bits)
    s = scales_gn.to(dtype).contiguous()
    if zeros_gn is None:
        zeros_gn = torch.full_like(scales_gn, float(1 << (bits - 1)), dtype=torch.float32)
    z = (zeros_gn.float() + zero_bias(bits, dtype)).to(dtype).contiguous()
    return qc, s, z


def dequantize_canonical(qc, scales, zeros, bits: int, group: int) -> torch.Tensor:
    """fp32 ``[.., N, K]`` weights from the canonical layout (the oracle the kernel is tested against)."""
    q = unpack_canonical(qc, bits).float()
    z = zeros.float() - zero_bias(bits, scales.dtype)
    s = scales.float()
    s_nk = s.transpose(-1, -2).repeat_interleave(group, dim=-1)
    z_nk = z.transpose(-1, -2).repeat_interleave(group, dim=-1)
    return (q - z_nk) * s_nk


def quantize_weight(w_nk: torch.Tensor, bits: int, group: int, sym: bool = False):
    """Round-to-nearest group quantisation of ``w [N,K]`` (tests, dummy weights): values, scales, zeros."""
    N, K = w_nk.shape[-2:]
    wg = w_nk.float().reshape(*w_nk.shape[:-1], K // group, group)
    qmax = (1 << bits) - 1
    if sym:
        s = wg.abs().amax(-1).clamp_min(1e-8) / (qmax // 2)
        z = torch.full_like(s, float(1 << (bits - 1)))
    else:
        mx, mn = wg.amax(-1), wg.amin(-1)
        s = ((mx - mn) / qmax).clamp_min(1e-8)
        z = torch.round(-mn / s).clamp(0, qmax)
    q = torch.clamp(torch.round(wg / s.unsqueeze(-1)) + z.unsqueeze(-1), 0, qmax).to(torch.uint8)
    return q.reshape(w_nk.shape), s.transpose(-1, -2).contiguous(), z.transpose(-1, -2).contiguous()


# ----------------------------------------------------------------------------- checkpoint formats
def gptq_to_values(qweight, qzeros, bits: int, zero_plus_one: bool = True):
    """GPTQ: ``qweight int32 [K/pack, N]`` (packed along K), ``qzeros int32 [K/g, N/pack]`` (packed along N)."""
    q_kn = unpack_int32(qweight, bits, 0)
    z = unpack_int32(qzeros, bits, 1).to(torch.int32)
    if zero_plus_one:      # v1 checkpoints store zero - 1
        z = (z + 1) & ((1 << bits) - 1) if bits < 8 else z + 1
    return q_kn.transpose(0, 1).contiguous(), z


def awq_to_values(qweight, qzeros, bits: int = 4):
    """AWQ: ``qweight int32 [K, N/8]``, ``qzeros int32 [K/g, N/8]``, both packed along N in AWQ order."""
    assert bits == 4
    rev = torch.tensor(_AWQ_REVERSE, device=qweight.device)

    def un(t):
        v = unpack_int32(t, 4, 1)
        return v.reshape(v.shape[0], -1, 8)[:, :, rev].reshape(v.shape[0], -1)

    return un(qweight).transpose(0, 1).contiguous(), un(qzeros).to(torch.int32)


def ct_to_values(weight_packed, weight_zero_point, bits: int):
    """compressed-tensors pack-quantized: ``weight_packed int32 [N, K/pack]`` holding value + 2^(bits-1)
    offsets; optional ``weight_zero_point int32 [N/pack, K/g]`` packed along N."""
    q_nk = unpack_int32(weight_packed, bits, 1)
    z = None
    if weight_zero_point is not None:
        z = unpack_int32(weight_zero_point, bits, 0).to(torch.int32).transpose(0, 1).contiguous()   # [K/g, N]
    return q_nk, z


# ----------------------------------------------------------------------------- linear method
class WNA16LinearMethod(LinearMethodBase):
    """fmt: "gptq" | "awq" | "ct" (compressed-tensors) | "canonical"."""

    def __init__(self, fmt: str, bits: int, group: int, sym: bool = False, desc_act: bool = False,
                 zero_plus_one: bool = True):
        self.fmt, self.bits, self.group_cfg, self.sym, self.desc_act = fmt, bits, group, sym, desc_act
        self.zero_plus_one = zero_plus_one

    def create_weights(self, layer, in_features, out_features, dtype):
        K, N, bits = in_features, out_features, self.bits
        g = K if self.group_cfg in (-1, None) else self.group_cfg
        while K % g:            # a row-parallel shard narrower than one group
            g //= 2
        layer.wq_group, layer.wq_bits = g, bits
        pack = 32 // bits
        i32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.int32), requires_grad=False)
        f16 = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype), requires_grad=False)

        def tag(p, out_dim, in_dim, block_n=1):
            p.output_dim, p.input_dim, p.block_n = out_dim, in_dim, block_n
            return p

        if self.fmt == "gptq":
            layer.qweight = tag(i32(K // pack, N), 1, 0)
            layer.qzeros = tag(i32(K // g, N // pack), 1, 0, pack)
            layer.scales = tag(f16(K // g, N), 1, 0)
            layer.g_idx = nn.Parameter(torch.arange(K, dtype=torch.int32) // g, requires_grad=False)
            layer.g_idx.output_dim, layer.g_idx.input_dim = 1, 0
        elif self.fmt == "awq":
            layer.qweight = tag(i32(K, N // pack), 1, 0, pack)
            layer.qzeros = tag(i32(K // g, N // pack), 1, 0, pack)
            layer.scales = tag(f16(K // g, N), 1, 0)
        elif self.fmt == "ct":
            layer.weight_packed = tag(i32(N, K // pack), 0, 1)
            layer.weight_scale = tag(f16(N, K // g), 0, 1)
            if not self.sym:
                layer.weight_zero_point = tag(i32(N // pack, K // g), 0, 1, pack)
        else:
            layer.qweight_c = nn.Parameter(torch.zeros(N, K * bits // 8, dtype=torch.uint8), requires_grad=False)
            layer.scales_c = f16(K // g, N)
            layer.zeros_c = f16(K // g, N)
        layer.wq_ready = self.fmt == "canonical"

    def process_weights_after_loading(self, layer) -> None:
        if getattr(layer, "wq_ready", True):
            return
        bits, dtype = self.bits, layer.dtype
        perm = None
        if self.fmt == "gptq":
            q_nk, z = gptq_to_values(layer.qweight.data, layer.qzeros.data, bits, self.zero_plus_one)
            scales = layer.scales.data
            g_idx = layer.g_idx.data.long()
            if self.desc_act and not torch.equal(g_idx, torch.arange(g_idx.numel(), device=g_idx.device) // layer.wq_group):
                perm = torch.argsort(g_idx, stable=True)
                q_nk = q_nk[:, perm]
            names = ("qweight", "qzeros", "scales", "g_idx")
        elif self.fmt == "awq":
            q_nk, z = awq_to_values(layer.qweight.data, layer.qzeros.data, bits)
            scales = layer.scales.data
            names = ("qweight", "qzeros", "scales")
        else:
            zp = getattr(layer, "weight_zero_point", None)
            q_nk, z = ct_to_values(layer.weight_packed.data, None if zp is None else zp.data, bits)
            scales = layer.weight_scale.data.transpose(0, 1).contiguous()
            names = ("weight_packed", "weight_scale", "weight_zero_point")
        if self.sym and self.fmt != "ct":
            z = None
        qc, s, zc = canonical_from_values(q_nk, scales, z, bits, dtype)
        for n in names:
            if hasattr(layer, n):
                delattr(layer, n)
        layer.qweight_c = nn.Parameter(qc, requires_grad=False)
        layer.scales_c = nn.Parameter(s, requires_grad=False)
        layer.zeros_c = nn.Parameter(zc, requires_grad=False)
        layer.act_perm = None if perm is None else perm.to(torch.int64)
        layer.wq_ready = True

    def apply(self, layer, x, bias=None, residual=None):
        perm = getattr(layer, "act_perm", None)
        if perm is not None:
            x = x.index_select(-1, perm.to(x.device))
        y = ops.wna16_gemm(x, layer.qweight_c, layer.scales_c, layer.zeros_c, layer.wq_bits, layer.wq_group, bias=bias)
        if residual is not None:
            y = y + residual
        return y


# ----------------------------------------------------------------------------- MoE method
class WNA16MoEMethod:
    """Experts with group-quantised weights.  Canonical storage: ``w13_q [E, 2I, H*bits/8]`` (gate / up rows
    interleaved so the GEMM epilogue applies SiLU-gate), ``w2_q [E, H, I*bits/8]`` and their
    ``[E, K/g, N]`` scales / zeros.  Checkpoint tensors arrive per expert in GPTQ / AWQ / compressed-tensors
    form and are converted as they are loaded.  ``act_int8`` (W4A8 checkpoints) keeps activations in 16 bit:
    the same kernel, no precision loss."""

    def __init__(self, fmt: str, bits: int, group: int, sym: bool = False, zero_plus_one: bool = True,
                 act_int8: bool = False):
        self.fmt, self.bits, self.group, self.sym, self.zero_plus_one = fmt, bits, group, sym, zero_plus_one
        self.act_int8 = act_int8

    def create_weights(self, layer, num_local, hidden, inter, dtype):
        b = self.bits
        g13 = hidden if self.group in (-1, None) else self.group
        g2 = inter if self.group in (-1, None) else min(self.group, inter)
        self.g13, self.g2, self.inter, self.hidden, self.dtype = g13, g2, inter, hidden, dtype
        u8 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.uint8), requires_grad=False)
        f16 = lambda *s: nn.Parameter(torch.ones(*s, dtype=dtype), requires_grad=False)
        layer.w13_q, layer.w2_q = u8(num_local, 2 * inter, hidden * b // 8), u8(num_local, hidden, inter * b // 8)
        layer.w13_s, layer.w13_z = f16(num_local, hidden // g13, 2 * inter), f16(num_local, hidden // g13, 2 * inter)
        layer.w2_s, layer.w2_z = f16(num_local, inter // g2, hidden), f16(num_local, inter // g2, hidden)
        self._staging: dict = {}

    # checkpoint tensors of one expert projection arrive one by one; convert when the set is complete
    def load_expert_tensor(self, layer, e: int, shard: str, kind: str, tensor: torch.Tensor) -> None:
        need = {"gptq": ("qweight", "qzeros", "scales"), "awq": ("qweight", "qzeros", "scales"),
                "ct": ("weight_packed", "weight_scale") + (() if self.sym else ("weight_zero_point",))}[self.fmt]
        if kind not in need:
            return
        st = self._staging.setdefault((e, shard), {})
        st[kind] = tensor
        if all(k in st for k in need):
            self._convert(layer, e, shard, st)
            del self._staging[(e, shard)]

    def _convert(self, layer, e, shard, st):
        b = self.bits
        if self.fmt == "gptq":
            q_nk, z = gptq_to_values(st["qweight"], st["qzeros"], b, self.zero_plus_one)
            s = st["scales"]
        elif self.fmt == "awq":
            q_nk, z = awq_to_values(st["qweight"], st["qzeros"], b)
            s = st["scales"]
        else:
            q_nk, z = ct_to_values(st["weight_packed"], st.get("weight_zero_point"), b)
            s = st["weight_scale"].transpose(0, 1).contiguous()
        if self.sym and self.fmt != "ct":
            z = None
        self.store_expert(layer, e, shard, q_nk, s, z)

    def store_expert(self, layer, e: int, shard: str, q_nk, scales_gn, zeros_gn) -> None:
        qc, s, z = canonical_from_values(q_nk, scales_gn, zeros_gn, self.bits, self.dtype)
        if shard == "w2":
            layer.w2_q.data[e].copy_(qc)
            layer.w2_s.data[e].copy_(s)
            layer.w2_z.data[e].copy_(z)
            return
        off = 0 if shard == "w1" else 1     # gate rows even, up rows odd
        layer.w13_q.data[e, off::2].copy_(qc)
        layer.w13_s.data[e, :, off::2].copy_(s)
        layer.w13_z.data[e, :, off::2].copy_(z)

    def apply(self, layer, x, topk_weights, topk_ids, shared_out=None):
        T, topk = x.shape[0], topk_ids.shape[1]
        from ..layers.moe_configs import try_get_optimal_moe_config

        # tuned (or heuristic) row-block size: small per-expert batches waste less of a tile
        tile = int(try_get_optimal_moe_config(T, layer.num_local, self.inter, self.hidden, topk, "w4a16")["token_tile"])
        sorted_ids, block_expert, total, inv = ops.moe_align_block_size(topk_ids, tile, layer.num_local,
                                                                        layer.expert_map, want_inverse=True)
        a = ops.moe_gather(x, sorted_ids, total, topk)
        h = ops.wna16_gemm(a, layer.w13_q, layer.w13_s, layer.w13_z, self.bits, self.g13, block_expert=block_expert,
                           total_padded=total, token_tile=tile, silu_gate=True)
        y = ops.wna16_gemm(h, layer.w2_q, layer.w2_s, layer.w2_z, self.bits, self.g2, block_expert=block_expert,
                           total_padded=total, token_tile=tile)
        return ops.moe_combine(y, topk_weights, inv, T, shared_out)


# ----------------------------------------------------------------------------- configs
class _WeightOnlyConfig:
    fmt = "gptq"

    def __init__(self, bits: int, group: int, sym: bool, desc_act: bool, ignored: list[str], zero_plus_one: bool = True):
        if bits not in (4, 8):
            raise ValueError(f"{bits}-bit weights are not supported (4 or 8)")
        self.bits, self.group, self.sym, self.desc_act, self.ignored = bits, group, sym, desc_act, ignored
        self.zero_plus_one = zero_plus_one

    def _skip(self, prefix: str) -> bool:
        return any(ig and ig in prefix for ig in self.ignored) or prefix.endswith("lm_head") or prefix.endswith(".gate")

    def get_linear_method(self, prefix: str) -> Optional[LinearMethodBase]:
        if self._skip(prefix):
            return None
        return WNA16LinearMethod(self.fmt, self.bits, self.group, self.sym, self.desc_act, self.zero_plus_one)

    def get_moe_method(self, prefix: str):
        return WNA16MoEMethod(self.fmt, self.bits, self.group, self.sym, self.zero_plus_one)


class GPTQConfig(_WeightOnlyConfig):
    """``{"quant_method": "gptq", "bits": 4, "group_size": 128, "desc_act": false, "sym": true}``."""
    fmt = "gptq"

    def __init__(self, cfg: dict):
        v2 = cfg.get("checkpoint_format") == "gptq_v2"
        super().__init__(int(cfg.get("bits", 4)), int(cfg.get("group_size", 128)), bool(cfg.get("sym", True)),
                         bool(cfg.get("desc_act", False)), list(cfg.get("modules_to_not_convert") or []), not v2)


class AWQConfig(_WeightOnlyConfig):
    """``{"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": true}``."""
    fmt = "awq"

    def __init__(self, cfg: dict):
        bits = int(cfg.get("bits", cfg.get("w_bit", 4)))
        if bits != 4:
            raise ValueError("AWQ checkpoints are 4-bit")
        super().__init__(bits, int(cfg.get("group_size", cfg.get("q_group_size", 128))), False, False,
                         list(cfg.get("modules_to_not_convert") or []))


class MoeWNA16Config(_WeightOnlyConfig):
    """``moe_wna16``: experts quantised (GPTQ or AWQ layout), everything else follows ``full_config``."""

    def __init__(self, cfg: dict):
        inner = (cfg.get("full_config") or cfg)
        self.fmt = "awq" if inner.get("quant_method", cfg.get("linear_quant_method", "gptq")) == "awq" else "gptq"
        super().__init__(int(cfg.get("bits", 4)), int(cfg.get("group_size", 128)), bool(cfg.get("sym", self.fmt == "gptq")),
                         False, list(cfg.get("modules_to_not_convert") or []))
        self.quantize_dense = bool(cfg.get("quantize_dense", True))

    def get_linear_method(self, prefix: str):
        return super().get_linear_method(prefix) if self.quantize_dense else None


class CompressedTensorsConfig:
    """compressed-tensors: dispatches per ``config_groups`` scheme - weight-only ``pack-quantized`` (WNA16),
    ``int-quantized`` W8A8 (static or dynamic per-token activations) and W4A8 experts."""

    def __init__(self, cfg: dict):
        self.ignored = list(cfg.get("ignore") or [])
        groups = cfg.get("config_groups") or {}
        grp = next(iter(groups.values()), {}) if groups else {}
        w = grp.get("weights") or {}
        a = grp.get("input_activations")
        self.bits = int(w.get("num_bits", 4))
        self.group = int(w.get("group_size") or -1)
        self.sym = bool(w.get("symmetric", True))
        self.strategy = w.get("strategy", "group")
        self.act_bits = int(a.get("num_bits", 16)) if a else 16
        self.act_dynamic = bool(a.get("dynamic", True)) if a else True
        self.act_sym = bool(a.get("symmetric", True)) if a else True
        self.format = cfg.get("format", "pack-quantized")

    def _skip(self, prefix: str) -> bool:
        return any(ig.replace("re:", "") in prefix for ig in self.ignored) or prefix.endswith("lm_head")

    @property
    def is_w8a8(self) -> bool:
        return self.bits == 8 and self.act_bits == 8

    def get_linear_method(self, prefix: str):
        if self._skip(prefix):
            return None
        if self.is_w8a8:
            from .int8 import Int8LinearMethod

            return Int8LinearMethod(static_act=not self.act_dynamic, act_sym=self.act_sym,
                                    per_channel=self.strategy == "channel")
        return WNA16LinearMethod("ct", self.bits, self.group, self.sym)

    def get_moe_method(self, prefix: str):
        if self.is_w8a8:
            from .int8 import Int8MoEMethod

            return Int8MoEMethod()
        if self.bits == 4 and self.act_bits == 8 and self.sym and (self.group in (-1, None) or self.strategy == "channel"):
            from .int8 import W4A8Int8MoEMethod      # channel-wise W4 + int8 activations: the integer tensor-core path

            return W4A8Int8MoEMethod(self.bits)
        return WNA16MoEMethod("ct", self.bits, self.group, self.sym, act_int8=self.act_bits == 8)


for _name, _cls in (("gptq", GPTQConfig), ("auto_gptq", GPTQConfig), ("awq", AWQConfig), ("auto_awq", AWQConfig),
                    ("moe_wna16", MoeWNA16Config), ("compressed_tensors", CompressedTensorsConfig)):
    register_quantization_config(_name)(_cls)
