"""TurboQuant KV cache (``csrc/tq_cache.cu``): 3-4 bit keys (Hadamard rotation + Lloyd-Max levels + stored norm, or
plain fp8) and 3-4 bit uniform values in one slot per (token, kv head), with the fp32 PyTorch statement of every
op (also the CPU path).

Presets (``--kv-cache-dtype``): ``turboquant_k8v4``, ``turboquant_4bit_nc``, ``turboquant_k3v4_nc``,
``turboquant_3bit_nc`` (``nc`` = the stored norm is corrected so that the reconstructed key keeps its length).
Cache: ``uint8 [blocks, block_size, kv_heads, slot_bytes]``, head_dim 128.

Parity: vllm_metax/v1/attention/backends/turboquant_attn.py:95-942 (backend, builder, impl) and the preset table of
upstream's quantization/turboquant/config.py; the store / decode kernels replace upstream's Triton ones.
"""
from __future__ import annotations

import functools
import math
from dataclasses import dataclass
from typing import Optional

import torch

D = 128
LEVELS = {
    4: (-2.7326, -2.0690, -1.6181, -1.2562, -0.9424, -0.6568, -0.3881, -0.1284,
        0.1284, 0.3881, 0.6568, 0.9424, 1.2562, 1.6181, 2.0690, 2.7326),
    3: (-2.1520, -1.3439, -0.7560, -0.2451, 0.2451, 0.7560, 1.3439, 2.1520),
}
PRESETS = {
    "turboquant_k8v4": (8, 4, False),
    "turboquant_4bit_nc": (4, 4, True),
    "turboquant_k3v4_nc": (3, 4, True),
    "turboquant_3bit_nc": (3, 3, True),
}


@dataclass(frozen=True)
class TqFormat:
    kbits: int
    vbits: int
    nc: bool

    @classmethod
    def from_name(cls, name: str) -> "TqFormat":
        if name not in PRESETS:
            raise ValueError(f"unknown TurboQuant preset {name!r}; valid: {', '.join(PRESETS)}")
        return cls(*PRESETS[name])

    @property
    def k_bytes(self) -> int:
        return 128 if self.kbits == 8 else self.kbits * 16

    @property
    def v_bytes(self) -> int:
        return self.vbits * 16

    @property
    def slot_bytes(self) -> int:
        return (self.k_bytes + self.v_bytes + 6 + 15) // 16 * 16

    @property
    def compression(self) -> float:
        return 2 * D * 2 / self.slot_bytes


def is_turboquant(cache_dtype: Optional[str]) -> bool:
    return bool(cache_dtype) and str(cache_dtype).startswith("turboquant")


def alloc_cache(num_blocks: int, block_size: int, kv_heads: int, fmt: TqFormat, device) -> torch.Tensor:
    return torch.zeros(num_blocks, block_size, kv_heads, fmt.slot_bytes, dtype=torch.uint8, device=device)


@functools.lru_cache(maxsize=None)
def hadamard(device: str = "cpu") -> torch.Tensor:
    """Orthonormal 128 x 128 Sylvester Hadamard matrix (symmetric, its own inverse)."""
    h = torch.ones(1, 1)
    while h.shape[0] < D:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / math.sqrt(D)).to(device)


# ------------------------------------------------------------------------------------------ fp32 statements
def _quantize_ref(k: torch.Tensor, v: torch.Tensor, fmt: TqFormat):
    """k, v [..., 128] -> dict of codes and metadata (the values the kernel stores, before bit packing)."""
    kf, vf = k.float(), v.float()
    out = {}
    if fmt.kbits == 8:
        out["k_fp8"] = kf.clamp(-448, 448).to(torch.float8_e4m3fn)
        out["k_norm"] = torch.ones(kf.shape[:-1])
    else:
        lv = torch.tensor(LEVELS[fmt.kbits])
        norm = kf.norm(dim=-1, keepdim=True)
        u = torch.where(norm > 0, kf / norm, torch.zeros_like(kf)) @ hadamard()
        z = u * math.sqrt(D)
        mid = (lv[1:] + lv[:-1]) / 2
        codes = (z[..., None] > mid).sum(-1)
        out["k_codes"] = codes
        ln = (lv[codes].pow(2).sum(-1, keepdim=True) / D).sqrt()
        stored = torch.where(ln > 0, norm / ln, norm) if fmt.nc else norm
        out["k_norm"] = stored[..., 0].half().float()
    vmax = (1 << fmt.vbits) - 1
    mn, mx = vf.amin(-1, keepdim=True), vf.amax(-1, keepdim=True)
    scale = ((mx - mn) / vmax).clamp_min(1e-8).half().float()
    zero = mn.half().float()
    out["v_codes"] = torch.round((vf - zero) / scale).clamp(0, vmax).long()
    out["v_scale"], out["v_zero"] = scale[..., 0], zero[..., 0]
    return out


def _dequant_from(qd: dict, fmt: TqFormat):
    if fmt.kbits == 8:
        k = qd["k_fp8"].float()
    else:
        lv = torch.tensor(LEVELS[fmt.kbits])
        k = (lv[qd["k_codes"]] / math.sqrt(D)) @ hadamard() * qd["k_norm"][..., None]
    v = qd["v_codes"].float() * qd["v_scale"][..., None] + qd["v_zero"][..., None]
    return k, v


def quant_dequant_ref(k: torch.Tensor, v: torch.Tensor, fmt: TqFormat):
    """What a reader of the cache sees for ``k, v [..., 128]`` (fp32)."""
    return _dequant_from(_quantize_ref(k.cpu(), v.cpu(), fmt), fmt)


def decode_attention_ref(q, k_hat, v_hat, seq_lens, scale):
    """q [B, Hq, 128]; k_hat / v_hat: per-sequence lists of the dequantised ``[L, Hkv, 128]``."""
    B, Hq, _ = q.shape
    out = torch.zeros(B, Hq, D)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        g = Hq // k_hat[b].shape[1]
        kk = k_hat[b][:L].repeat_interleave(g, 1)
        vv = v_hat[b][:L].repeat_interleave(g, 1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), kk) * scale
        out[b] = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vv)
    return out


# ------------------------------------------------------------------------------------------ ops
class _CpuCache:
    """CPU stand-in: the dequantised rows are kept beside the (unused) byte tensor, keyed by its storage."""
    store: dict = {}


def store(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, slot_mapping: torch.Tensor, fmt: TqFormat) -> None:
    """Quantise ``k, v [T, Hkv * 128]`` into the slots ``slot_mapping`` (negative: skipped)."""
    if cache.is_cuda:
        from .. import _custom_ops as ops

        ops.load_native()
        ops._launches += 1
        torch.ops.b200.tq_store(cache, k, v, slot_mapping.long().contiguous(), fmt.kbits, fmt.vbits, fmt.nc)
        return
    heads = cache.shape[2]
    n = slot_mapping.numel()
    kh, vh = quant_dequant_ref(k[:n].reshape(n, heads, D), v[:n].reshape(n, heads, D), fmt)
    side = _CpuCache.store.setdefault(cache.data_ptr(), {})
    for i, s in enumerate(slot_mapping.tolist()):
        if s >= 0:
            side[s] = (kh[i], vh[i])


def dequant(cache: torch.Tensor, slots: torch.Tensor, fmt: TqFormat, dtype=torch.bfloat16):
    """Slots -> ``(k, v) [n, Hkv, 128]`` in ``dtype`` (negative slots give zero rows)."""
    heads = cache.shape[2]
    n = slots.numel()
    if cache.is_cuda:
        from .. import _custom_ops as ops

        ops.load_native()
        k = torch.empty(n, heads, D, dtype=dtype, device=cache.device)
        v = torch.empty_like(k)
        ops._launches += 1
        torch.ops.b200.tq_dequant(k, v, cache, slots.long().contiguous(), fmt.kbits, fmt.vbits, fmt.nc)
        return k, v
    side = _CpuCache.store.get(cache.data_ptr(), {})
    k, v = torch.zeros(n, heads, D), torch.zeros(n, heads, D)
    for i, s in enumerate(slots.tolist()):
        if s >= 0 and s in side:
            k[i], v[i] = side[s]
    return k.to(dtype), v.to(dtype)


def _slots_of(block_table_row: torch.Tensor, L: int, block_size: int) -> torch.Tensor:
    t = torch.arange(L, device=block_table_row.device)
    return block_table_row[t // block_size].long() * block_size + t % block_size


def decode_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                     scale: float, fmt: TqFormat, num_splits: int = 0, out: Optional[torch.Tensor] = None):
    """One query token per sequence: ``q [B, Hq, 128]`` against the compressed cache -> ``[B, Hq, 128]``."""
    B, Hq, _ = q.shape
    if q.is_cuda:
        from .. import _custom_ops as ops

        ops.load_native()
        out = torch.empty_like(q) if out is None else out
        hkv = cache.shape[2]
        if num_splits <= 0:           # enough CTAs for the 148 SMs, at least 256 tokens per split
            max_len = int(cache.shape[1]) * block_table.shape[1]
            num_splits = max(1, min(16, (2 * 148) // max(1, B * hkv), max_len // 256))
        ws = torch.empty(num_splits * B * Hq * 129, dtype=torch.float32, device=q.device) if num_splits > 1 else None
        ops._launches += 1 + (num_splits > 1)
        torch.ops.b200.tq_decode(out, q.contiguous(), cache, block_table.int().contiguous(),
                                 seq_lens.int().contiguous(), ws, scale, num_splits, fmt.kbits, fmt.vbits, fmt.nc)
        return out
    ks, vs = [], []
    for b in range(B):
        k, v = dequant(cache, _slots_of(block_table[b], int(seq_lens[b]), cache.shape[1]), fmt, torch.float32)
        ks.append(k)
        vs.append(v)
    res = decode_attention_ref(q, ks, vs, seq_lens, scale).to(q.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res
