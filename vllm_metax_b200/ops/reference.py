"""Plain PyTorch (fp32 math) implementations of every op in the framework.

Each function here plays three roles: it is the numerical oracle the CUDA
kernels are tested against, it is the execution path on CPU tensors (the
plumbing configuration runs the whole engine through these), and it documents
the exact semantics of the op.  None of them is used on the GPU hot path.

Layouts
-------
* paged KV cache (bf16/fp16/fp8): ``[num_blocks, 2, block_size, num_kv_heads, head_dim]``
  (K at index 0 of dim 1, V at index 1).
* int8 / fp8 per-token-head cache: same shape in int8/e4m3 plus
  ``kv_scales [num_blocks, 2, block_size, num_kv_heads]`` f32 (symmetric).
* MLA latent cache: ``[num_blocks, block_size, 576]`` bf16 or
  ``[num_blocks, block_size, 656]`` uint8 ("fp8_ds_mla": 512 e4m3, 4 f32
  scales, 64 bf16 rope) - vllm_metax/v1/attention/backends/mla/flashmla_sparse.py:72-93.
* indexer K cache: ``uint8 [num_blocks, block_size*132]`` block-planar
  (``block_size*128`` e4m3 bytes then ``block_size`` f32 scales) -
  csrc/libtorch_stable/cache_kernels.cu:545-605 of the reference.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8_DTYPE = torch.float8_e4m3fn


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w.  Ref kernel: layernorm_kernels.cu:15."""
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """residual' = x + residual (rounded to dtype); y = rms_norm(residual').

    Returns ``(y, residual')``.  Ref kernel: layernorm_kernels.cu:100,172.
    """
    r = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(r, weight, eps), r


def gemma_rms_norm(x, weight, eps):
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * (1.0 + weight.float())).to(x.dtype)


def rms_norm_gated(x, gate, weight, eps):
    """RMSNorm(x) * silu(gate) (Mamba2 / GDN style gated norm)."""
    return (rms_norm(x, weight, eps).float() * F.silu(gate.float())).to(x.dtype)


def layer_norm(x, weight, bias, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


# --------------------------------------------------------------------------- rope
def build_rope_cache(rot_dim: int, max_pos: int, base: float, dtype=torch.float32,
                     scaling: Optional[dict] = None) -> torch.Tensor:
    """cos/sin table ``[max_pos, rot_dim]`` = ``[cos(rot/2) | sin(rot/2)]``.

    ``scaling`` supports ``{"type": "linear"|"llama3"|"yarn", ...}``.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    mscale = 1.0
    if scaling:
        t = scaling.get("rope_type", scaling.get("type", "default"))
        if t == "linear":
            inv_freq = inv_freq / float(scaling["factor"])
        elif t == "llama3":
            factor = float(scaling["factor"])
            lo = float(scaling.get("low_freq_factor", 1.0))
            hi = float(scaling.get("high_freq_factor", 4.0))
            old = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = ((old / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > old / lo, inv_freq / factor, inv_freq)
            mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
            is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
            inv_freq = torch.where(is_mid, mid, scaled)
        elif t in ("yarn", "deepseek_yarn"):
            factor = float(scaling["factor"])
            old = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast = float(scaling.get("beta_fast", 32))
            beta_slow = float(scaling.get("beta_slow", 1))

            def corr_dim(n_rot):
                return (rot_dim * math.log(old / (n_rot * 2 * math.pi))) / (2 * math.log(base))

            low = max(math.floor(corr_dim(beta_fast)), 0)
            high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
            ramp = torch.clamp((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / max(high - low, 1e-3), 0, 1)
            inv_mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - inv_mask) + inv_freq * inv_mask

            def get_mscale(scale, m):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

            ms = float(scaling.get("mscale", 1))
            ms_all = float(scaling.get("mscale_all_dim", 0))
            if t == "deepseek_yarn" or "mscale_all_dim" in scaling:
                mscale = get_mscale(factor, ms) / get_mscale(factor, ms_all) if ms_all else get_mscale(factor, ms)
            else:
                mscale = get_mscale(factor, 1.0)
    t_pos = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t_pos, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).to(dtype)


def rotary_embedding(positions: torch.Tensor, q: torch.Tensor, k: Optional[torch.Tensor], head_size: int,
                     cos_sin_cache: torch.Tensor, is_neox: bool = True, rot_offset: int = 0,
                     inverse: bool = False):
    """RoPE on ``q [T, Hq*head_size]`` and ``k [T, Hk*head_size]``; returns new tensors.

    NeoX style rotates (x[:r/2], x[r/2:]); GPT-J style rotates interleaved pairs.
    ``rot_offset`` is the first rotated element inside each head; ``inverse``
    applies the transposed rotation.  Ref kernel: pos_encoding_kernels.cu:77.
    """
    rot = cos_sin_cache.shape[-1]
    cs = cos_sin_cache.float()[positions.long()]
    cos, sin = cs[:, : rot // 2], cs[:, rot // 2:]
    if inverse:
        sin = -sin

    def apply(x):
        if x is None:
            return None
        T = x.shape[0]
        xh = x.float().reshape(T, -1, head_size).clone()
        xr = xh[..., rot_offset: rot_offset + rot]
        c, s = cos[:, None, :], sin[:, None, :]
        if is_neox:
            x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
            o = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        else:
            x1, x2 = xr[..., 0::2], xr[..., 1::2]
            o = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
        xh[..., rot_offset: rot_offset + rot] = o
        return xh.reshape(x.shape).to(x.dtype)

    return apply(q), apply(k)


# --------------------------------------------------------------------------- activations
def _act(name: str, x: torch.Tensor, **kw) -> torch.Tensor:
    if name == "silu":
        return F.silu(x)
    if name == "gelu":
        return F.gelu(x)
    if name == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if name == "relu2":
        return F.relu(x) ** 2
    if name == "fatrelu":
        return torch.where(x > kw.get("threshold", 0.0), x, torch.zeros_like(x))
    if name == "gelu_new":
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))
    if name == "gelu_fast":
        return 0.5 * x * (1.0 + torch.tanh(x * 0.7978845608 * (1.0 + 0.044715 * x * x)))
    if name == "gelu_quick":
        return x * torch.sigmoid(1.702 * x)
    raise ValueError(name)


def act_and_mul(x: torch.Tensor, act: str = "silu", **kw) -> torch.Tensor:
    """out = act(x[..., :d]) * x[..., d:].  Ref kernel: activation_kernels.cu:102."""
    d = x.shape[-1] // 2
    return (_act(act, x[..., :d].float(), **kw) * x[..., d:].float()).to(x.dtype)


def silu_and_mul(x):
    return act_and_mul(x, "silu")


def mul_and_silu(x):
    d = x.shape[-1] // 2
    return (x[..., :d].float() * F.silu(x[..., d:].float())).to(x.dtype)


def swigluoai_and_mul(x, alpha: float = 1.702, limit: float = 7.0):
    """gate/up interleaved; gate clamped to <=limit, up to [-limit, limit];
    out = gate*sigmoid(alpha*gate) * (up+1).  Ref: activation_kernels.cu:412."""
    g = x[..., 0::2].float().clamp(max=limit)
    u = x[..., 1::2].float().clamp(min=-limit, max=limit)
    return ((u + 1.0) * g * torch.sigmoid(alpha * g)).to(x.dtype)


def swiglustep_and_mul(x, limit: float = 7.0):
    """Clamped SwiGLU of the "step" family: silu(gate).clamp(max=limit) * up.clamp(+-limit)."""
    d = x.shape[-1] // 2
    g = F.silu(x[..., :d].float()).clamp(max=limit)
    u = x[..., d:].float().clamp(min=-limit, max=limit)
    return (g * u).to(x.dtype)


def activation(x, act: str):
    return _act(act, x.float()).to(x.dtype)


# --------------------------------------------------------------------------- quantisation
def to_fp8(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)


def static_scaled_fp8_quant(x, scale):
    return to_fp8(x.float() / scale.float())


def dynamic_scaled_fp8_quant(x):
    """Per-tensor dynamic: scale = amax/448."""
    scale = (x.float().abs().max() / FP8_MAX).clamp(min=1e-12)
    return to_fp8(x.float() / scale), scale.reshape(1)


def dynamic_per_token_scaled_fp8_quant(x, scale_ub: Optional[float] = None):
    amax = x.float().abs().amax(dim=-1, keepdim=True)
    if scale_ub is not None:
        amax = amax.clamp(max=scale_ub)
    scale = (amax / FP8_MAX).clamp(min=1.0 / (FP8_MAX * 512.0))
    return to_fp8(x.float() / scale), scale


def _ue8m0_round(scale: torch.Tensor) -> torch.Tensor:
    return torch.exp2(torch.ceil(torch.log2(scale.clamp(min=1e-30))))


def per_token_group_quant_fp8(x, group_size: int = 128, eps: float = 1e-10, ue8m0: bool = False):
    """1 x group_size dynamic fp8; returns ``(q [.., K], scales [.., K/g] f32)``.

    Ref kernel: quantization/w8a8/fp8/per_token_group_quant.cu:100.
    """
    shp = x.shape
    xg = x.float().reshape(*shp[:-1], shp[-1] // group_size, group_size)
    amax = xg.abs().amax(dim=-1, keepdim=True).clamp(min=eps)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = _ue8m0_round(scale)
    q = to_fp8(xg / scale).reshape(shp)
    return q, scale.squeeze(-1)


def per_token_group_quant_int8(x, group_size: int = 128, eps: float = 1e-10):
    shp = x.shape
    xg = x.float().reshape(*shp[:-1], shp[-1] // group_size, group_size)
    amax = xg.abs().amax(dim=-1, keepdim=True).clamp(min=eps)
    scale = amax / 127.0
    q = torch.round(xg / scale).clamp(-128, 127).to(torch.int8).reshape(shp)
    return q, scale.squeeze(-1)


def scaled_int8_quant(x, scale: Optional[torch.Tensor] = None, azp: Optional[torch.Tensor] = None,
                      symmetric: bool = True):
    """Static / dynamic-per-token int8 quantisation, symmetric or with zero point.

    Returns ``(q, scale, azp_or_None)``.  Ref: quantization/w8a8/int8/scaled_quant.cu:100-212.
    """
    xf = x.float()
    if scale is not None:  # static
        if symmetric:
            q = torch.round(xf / scale.float()).clamp(-128, 127).to(torch.int8)
            return q, scale, None
        q = (torch.round(xf / scale.float()) + azp.float()).clamp(-128, 127).to(torch.int8)
        return q, scale, azp
    if symmetric:
        amax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10)
        s = amax / 127.0
        return torch.round(xf / s).clamp(-128, 127).to(torch.int8), s, None
    mx = xf.amax(dim=-1, keepdim=True)
    mn = xf.amin(dim=-1, keepdim=True)
    s = ((mx - mn) / 255.0).clamp(min=1e-10)
    zp = torch.round(-128.0 - mn / s)
    q = (torch.round(xf / s) + zp).clamp(-128, 127).to(torch.int8)
    return q, s, zp.to(torch.int32)


def rms_norm_static_fp8_quant(x, weight, scale, eps):
    return to_fp8(rms_norm(x, weight, eps).float() / scale.float())


def rms_norm_dynamic_per_token_quant(x, weight, eps, quant_dtype=FP8_DTYPE, residual=None, scale_ub=None):
    if residual is not None:
        y, residual = fused_add_rms_norm(x, residual, weight, eps)
    else:
        y = rms_norm(x, weight, eps)
    if quant_dtype == torch.int8:
        q, s, _ = scaled_int8_quant(y)
    else:
        q, s = dynamic_per_token_scaled_fp8_quant(y, scale_ub)
    return q, s, residual


def rms_norm_per_block_quant(x, weight, eps, group_size=128, residual=None, ue8m0=False):
    if residual is not None:
        y, residual = fused_add_rms_norm(x, residual, weight, eps)
    else:
        y = rms_norm(x, weight, eps)
    q, s = per_token_group_quant_fp8(y, group_size, ue8m0=ue8m0)
    return q, s, residual


def silu_and_mul_quant(x, scale):
    return static_scaled_fp8_quant(silu_and_mul(x), scale)


def silu_and_mul_per_block_quant(x, group_size=128, ue8m0=False):
    return per_token_group_quant_fp8(silu_and_mul(x), group_size, ue8m0=ue8m0)


# --------------------------------------------------------------------------- GEMMs
def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``a [M,K] @ w[N,K]^T (+bias)`` with fp32 accumulation."""
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or a.dtype)


def dequant_block_fp8_weight(wq: torch.Tensor, scale_inv: torch.Tensor, block: Sequence[int] = (128, 128)):
    """``wq [N,K]`` e4m3 with ``scale_inv [ceil(N/bn), ceil(K/bk)]`` -> fp32."""
    N, K = wq.shape[-2:]
    bn, bk = block
    s = scale_inv.float().repeat_interleave(bn, dim=-2)[..., :N, :].repeat_interleave(bk, dim=-1)[..., :K]
    return wq.float() * s


def fp8_block_scaled_mm(aq, a_scale, wq, w_scale_inv, out_dtype=torch.bfloat16, block=(128, 128)):
    """Block-scaled fp8 GEMM: act 1x128 scales ``[M, K/128]``, weight 128x128 scales.

    Semantics of ``cutlass_fp8_block_scaled_mm`` as used at
    vllm_metax/model_executor/layers/quantization/_cutlass_ops.py:23-38.
    """
    K = aq.shape[-1]
    a = aq.float() * a_scale.float().repeat_interleave(block[1], dim=-1)[..., :K]
    w = dequant_block_fp8_weight(wq, w_scale_inv, block)
    return (a @ w.t()).to(out_dtype)


def scaled_mm(aq, wq, a_scale, w_scale, out_dtype=torch.bfloat16, bias=None, azp_adj=None, azp=None):
    """int8/fp8 GEMM with per-row(token) x per-column(channel) scales, optional bias and
    asymmetric zero-point correction ``- azp * azp_adj`` (azp_adj = column sums of W).

    Epilogue contract of csrc/cutlass_extensions (ScaledEpilogue[Bias][Azp[Token]]).
    """
    acc = aq.float() @ wq.float().t()
    if azp_adj is not None:
        if azp is not None:  # per-token azp
            acc = acc - azp.float().reshape(-1, 1) * azp_adj.float().reshape(1, -1)
        else:  # per-tensor azp already folded into azp_adj
            acc = acc - azp_adj.float().reshape(1, -1)
    y = acc * a_scale.float().reshape(-1, 1) * w_scale.float().reshape(1, -1)
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


# --------------------------------------------------------------------------- KV cache ops
def reshape_and_cache(key, value, kv_cache, slot_mapping, kv_scales=None, k_scale: float = 1.0,
                      v_scale: float = 1.0):
    """Scatter ``key/value [T, Hkv, D]`` into the paged cache at ``slot_mapping``
    (slot = block*block_size + offset; negative = skip).

    bf16/fp16 cache: copy.  fp8 cache without ``kv_scales``: static per-tensor
    scale.  int8/fp8 cache with ``kv_scales``: per-(token, head) symmetric scale
    ``amax/127`` (int8) or ``amax/448`` (fp8) stored in ``kv_scales``.
    Ref kernels: cache_kernels.cu:310-395, triton_reshape_and_cache_flash_per_token_head_quant.
    """
    nb, _, bs, H, D = kv_cache.shape
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    b, o = slots // bs, slots % bs
    for idx, (src, st) in enumerate(((key, k_scale), (value, v_scale))):
        s = src[valid].float()
        if kv_scales is not None:
            qmax = 127.0 if kv_cache.dtype == torch.int8 else FP8_MAX
            sc = (s.abs().amax(dim=-1) / qmax).clamp(min=1e-8)
            q = s / sc[..., None]
            if kv_cache.dtype == torch.int8:
                q = torch.round(q).clamp(-128, 127)
            kv_cache[b, idx, o] = q.to(kv_cache.dtype) if kv_cache.dtype == torch.int8 else to_fp8(q)
            kv_scales[b, idx, o] = sc
        elif kv_cache.dtype == FP8_DTYPE:
            kv_cache[b, idx, o] = to_fp8(s / st)
        else:
            kv_cache[b, idx, o] = s.to(kv_cache.dtype)


def gather_paged_kv(kv_cache, block_table_row, kv_len, kv_scales=None, k_scale=1.0, v_scale=1.0):
    """Contiguous fp32 ``(K, V) [kv_len, Hkv, D]`` of one sequence."""
    nb, _, bs, H, D = kv_cache.shape
    nblk = (kv_len + bs - 1) // bs
    blocks = block_table_row[:nblk].long()
    kv = kv_cache[blocks].float()  # [nblk, 2, bs, H, D]
    if kv_scales is not None:
        kv = kv * kv_scales[blocks].float()[..., None]
    k = kv[:, 0].reshape(-1, H, D)[:kv_len]
    v = kv[:, 1].reshape(-1, H, D)[:kv_len]
    if kv_scales is None and kv_cache.dtype == FP8_DTYPE:
        k, v = k * k_scale, v * v_scale
    return k, v


def copy_blocks(kv_caches: Sequence[torch.Tensor], src_to_dst: torch.Tensor):
    for c in kv_caches:
        c[src_to_dst[:, 1].long()] = c[src_to_dst[:, 0].long()]


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor):
    dst[src_to_dst[:, 1].long()] = src[src_to_dst[:, 0].long()].to(dst.device)


def convert_fp8(dst, src, scale: float = 1.0):
    if dst.dtype == FP8_DTYPE:
        dst.copy_(to_fp8(src.float() / scale))
    else:
        dst.copy_((src.float() * scale).to(dst.dtype))


# --------------------------------------------------------------------------- attention
def attention_core(q, k, v, scale, causal_offset: Optional[int] = None, window: int = -1,
                   softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                   alibi_slopes: Optional[torch.Tensor] = None):
    """Dense softmax attention for one sequence.

    ``q [Lq, Hq, D]``, ``k [Lk, Hkv, D]``, ``v [Lk, Hkv, Dv]`` (fp32).  Query row i
    sits at absolute position ``causal_offset + i`` and sees keys ``<=`` that
    position (``None`` = non-causal); ``window`` > 0 keeps only the last ``window``
    positions; ``sinks [Hq]`` adds one extra logit per head to the softmax
    denominator.  Returns ``(out [Lq,Hq,Dv], lse [Hq,Lq])``.
    """
    Lq, Hq, D = q.shape
    Lk, Hkv, _ = k.shape
    g = Hq // Hkv
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    kpos = torch.arange(Lk, device=q.device)[None, :]
    if causal_offset is not None:
        qpos = (causal_offset + torch.arange(Lq, device=q.device))[:, None]
    else:
        qpos = torch.full((Lq, 1), Lk - 1, device=q.device)
    if alibi_slopes is not None:
        s = s + alibi_slopes.float()[:, None, None] * (kpos - qpos)[None].float()
    mask = torch.zeros(Lq, Lk, dtype=torch.bool, device=q.device)
    if causal_offset is not None:
        mask |= kpos > qpos
    if window is not None and window > 0:
        mask |= kpos <= qpos - window
    s = s.masked_fill(mask[None], float("-inf"))
    if sinks is not None:
        s_ext = torch.cat([s, sinks.float()[:, None, None].expand(Hq, Lq, 1)], dim=-1)
        lse = torch.logsumexp(s_ext, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    out = torch.einsum("hqk,khd->qhd", p, vv)
    return out, lse


def paged_attention(q, kv_cache, block_table, seq_lens, query_start_loc, scale, *, kv_scales=None,
                    window: int = -1, softcap: float = 0.0, sinks=None, alibi_slopes=None,
                    k_scale: float = 1.0, v_scale: float = 1.0, causal: bool = True, return_lse: bool = False):
    """Varlen attention over the paged cache (prefill, chunked prefill and decode).

    ``q [T, Hq, D]`` holds the new tokens of every sequence back to back
    (``query_start_loc [B+1]``); sequence ``b`` has ``seq_lens[b]`` tokens in the
    cache *including* its new tokens, which must already have been written.
    Replaces flash_attn_varlen_func(block_table=...) / flash_attn_with_kvcache
    at vllm_metax/v1/attention/backends/flash_attn.py:1302-1355.
    """
    T, Hq, D = q.shape
    out = torch.zeros(T, Hq, kv_cache.shape[-1], dtype=torch.float32, device=q.device)
    lse_all = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    B = seq_lens.shape[0]
    qsl = query_start_loc.tolist()
    sl = seq_lens.tolist()
    for b in range(B):
        s0, s1 = qsl[b], qsl[b + 1]
        if s1 <= s0:
            continue
        k, v = gather_paged_kv(kv_cache, block_table[b], sl[b], kv_scales, k_scale, v_scale)
        o, lse = attention_core(q[s0:s1].float(), k, v, scale,
                                causal_offset=(sl[b] - (s1 - s0)) if causal else None,
                                window=window, softcap=softcap, sinks=sinks, alibi_slopes=alibi_slopes)
        out[s0:s1] = o
        lse_all[:, s0:s1] = lse
    out = out.to(q.dtype)
    return (out, lse_all) if return_lse else out


def merge_attn_states(prefix_out, prefix_lse, suffix_out, suffix_lse):
    """LSE-weighted merge of two partial attention results.

    ``*_out [T,H,D]``, ``*_lse [H,T]``; returns ``(out, lse)``.
    Ref kernel: attention/merge_attn_states.cu:19-130.
    """
    p_lse = prefix_lse.float().t()[..., None]
    s_lse = suffix_lse.float().t()[..., None]
    p_lse = torch.where(torch.isinf(p_lse) & (p_lse > 0), torch.full_like(p_lse, float("-inf")), p_lse)
    s_lse = torch.where(torch.isinf(s_lse) & (s_lse > 0), torch.full_like(s_lse, float("-inf")), s_lse)
    mx = torch.maximum(p_lse, s_lse)
    mx_safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    pw, sw = torch.exp(p_lse - mx_safe), torch.exp(s_lse - mx_safe)
    tot = (pw + sw)
    tot_safe = tot.clamp(min=1e-30)
    out = (prefix_out.float() * pw + suffix_out.float() * sw) / tot_safe
    lse = (torch.log(tot_safe) + mx_safe).squeeze(-1).t()
    lse = torch.where(tot.squeeze(-1).t() == 0, torch.full_like(lse, float("-inf")), lse)
    return out.to(prefix_out.dtype), lse


# --------------------------------------------------------------------------- MLA
def concat_and_cache_mla(kv_c, k_pe, mla_cache, slot_mapping):
    """Write ``[kv_c(512) | k_pe(64)]`` records.  bf16 cache ``[nb, bs, 576]`` or the
    656-byte fp8_ds_mla record.  Ref kernels: cache_kernels.cu:398, :442-541."""
    nb, bs = mla_cache.shape[:2]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    b, o = slots // bs, slots % bs
    if mla_cache.dtype != torch.uint8:
        mla_cache[b, o] = torch.cat([kv_c[valid], k_pe[valid]], dim=-1).to(mla_cache.dtype)
        return
    rec = pack_ds_mla(kv_c[valid], k_pe[valid])
    mla_cache[b, o] = rec


def pack_ds_mla(kv_c: torch.Tensor, k_pe: torch.Tensor) -> torch.Tensor:
    """``[T,512]`` + ``[T,64]`` -> ``uint8 [T,656]`` (512 e4m3 | 4 f32 scale | 64 bf16)."""
    T = kv_c.shape[0]
    x = kv_c.float().reshape(T, 4, 128)
    scale = (x.abs().amax(dim=-1) / FP8_MAX).clamp(min=1e-12)  # [T,4]
    q = to_fp8(x / scale[..., None]).reshape(T, 512)
    rec = torch.empty(T, 656, dtype=torch.uint8, device=kv_c.device)
    rec[:, :512] = q.view(torch.uint8)
    rec[:, 512:528] = scale.float().contiguous().view(torch.uint8).reshape(T, 16)
    rec[:, 528:] = k_pe.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(T, 128)
    return rec


def unpack_ds_mla(rec: torch.Tensor) -> torch.Tensor:
    """``uint8 [..., 656]`` -> fp32 ``[..., 576]``."""
    shp = rec.shape[:-1]
    r = rec.reshape(-1, 656)
    q = r[:, :512].contiguous().view(FP8_DTYPE).float().reshape(-1, 4, 128)
    sc = r[:, 512:528].contiguous().view(torch.float32).reshape(-1, 4, 1)
    pe = r[:, 528:].contiguous().view(torch.bfloat16).float()
    return torch.cat([(q * sc).reshape(-1, 512), pe], dim=-1).reshape(*shp, 576)


def gather_mla_cache(mla_cache, block_table_row, kv_len):
    nb, bs = mla_cache.shape[:2]
    nblk = (kv_len + bs - 1) // bs
    rows = mla_cache[block_table_row[:nblk].long()].reshape(nblk * bs, -1)[:kv_len]
    if mla_cache.dtype == torch.uint8:
        return unpack_ds_mla(rows)
    return rows.float()


def mla_decode(q, mla_cache, block_table, seq_lens, scale, kv_lora_rank: int = 512,
               query_start_loc=None, topk_indices: Optional[torch.Tensor] = None):
    """Absorbed MLA (MQA over the latent cache).

    ``q [T, H, 576]`` (``q_nope @ W_UK`` | ``q_pe``); output ``[T, H, 512]`` and
    ``lse [H, T]``.  With ``topk_indices [T, topk]`` (per-request token positions,
    -1 = none) only those cache entries are attended (DeepSeek sparse attention);
    otherwise row t of sequence b sees positions ``<= seq_len - q_len + i``.
    Semantics of flash_mla_with_kvcache / flash_mla_sparse_fwd
    (vllm_metax/v1/attention/ops/flashmla.py:109-139).
    """
    T, H, Dq = q.shape
    B = seq_lens.shape[0]
    if query_start_loc is None:
        query_start_loc = torch.arange(B + 1, device=q.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    out = torch.zeros(T, H, kv_lora_rank, dtype=torch.float32, device=q.device)
    lse_all = torch.full((H, T), float("-inf"), dtype=torch.float32, device=q.device)
    for b in range(B):
        s0, s1 = qsl[b], qsl[b + 1]
        if s1 <= s0:
            continue
        kv = gather_mla_cache(mla_cache, block_table[b], sl[b])  # [L,576]
        qq = q[s0:s1].float()
        s = torch.einsum("qhd,kd->hqk", qq, kv) * scale
        Lq, L = s1 - s0, sl[b]
        kpos = torch.arange(L, device=q.device)[None, :]
        qpos = (L - Lq + torch.arange(Lq, device=q.device))[:, None]
        mask = kpos > qpos
        if topk_indices is not None:
            idx = topk_indices[s0:s1].long()
            sel = torch.zeros(Lq, L + 1, dtype=torch.bool, device=q.device)
            sel.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, L)).clamp(max=L), True)
            mask = mask | ~sel[:, :L]
        s = s.masked_fill(mask[None], float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        p = torch.nan_to_num(torch.exp(s - lse[..., None]), nan=0.0)
        out[s0:s1] = torch.einsum("hqk,kd->qhd", p, kv[:, :kv_lora_rank])
        lse_all[:, s0:s1] = lse
    return out.to(q.dtype), lse_all


def concat_mla_q(ql_nope, q_pe):
    return torch.cat([ql_nope, q_pe], dim=-1)


# --------------------------------------------------------------------------- DSA indexer
def indexer_k_quant_and_cache(k, idx_cache, slot_mapping, quant_block: int = 128, ue8m0: bool = False,
                              int8: bool = False):
    """Quantise indexer keys ``k [T,128]`` to e4m3 + one f32 scale and insert into the
    block-planar cache ``uint8 [nb, bs*(128+4)]``.  Ref: cache_kernels.cu:545-605."""
    nb = idx_cache.shape[0]
    D = k.shape[-1]
    bs = idx_cache.shape[1] // (D + 4) if idx_cache.dim() == 2 else idx_cache.shape[1]
    flat = idx_cache.reshape(nb, -1)
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    b, o = slots // bs, slots % bs
    x = k[valid].float()
    scale = (x.abs().amax(dim=-1) / (127.0 if int8 else FP8_MAX)).clamp(min=1e-10)
    if ue8m0:
        scale = _ue8m0_round(scale)
    if int8:      # V4 indexer: int8 keys, same block-planar layout
        q = torch.round(x / scale[:, None]).clamp(-127, 127).to(torch.int8).view(torch.uint8)
    else:
        q = to_fp8(x / scale[:, None]).view(torch.uint8)
    sb = scale.float().contiguous().view(torch.uint8).reshape(-1, 4)
    cols = o[:, None] * D + torch.arange(D, device=k.device)[None]
    flat[b[:, None], cols] = q
    scols = bs * D + o[:, None] * 4 + torch.arange(4, device=k.device)[None]
    flat[b[:, None], scols] = sb


def gather_indexer_k(idx_cache, block_table_row, kv_len, D: int = 128, int8: bool = False):
    """Returns fp32 ``(k_q [L,128] (dequantised values *without* scale), scale [L])``."""
    nb = idx_cache.shape[0]
    flat = idx_cache.reshape(nb, -1)
    bs = flat.shape[1] // (D + 4)
    nblk = (kv_len + bs - 1) // bs
    blk = flat[block_table_row[:nblk].long()]
    kq = blk[:, : bs * D].contiguous().view(torch.int8 if int8 else FP8_DTYPE).float().reshape(nblk * bs, D)[:kv_len]
    sc = blk[:, bs * D:].contiguous().view(torch.float32).reshape(nblk * bs)[:kv_len]
    return kq, sc


def mqa_logits(q, k, k_scale, weights, ks, ke):
    """``logits[m,n] = sum_h w[m,h] * relu(q[m,h,:] . k[n,:]) * k_scale[n]`` within the
    row window ``[ks[m], ke[m])`` else -inf.  q ``[M,Hi,128]`` (fp8 values as float),
    k ``[N,128]``, weights ``[M,Hi]``.  Semantics of deep_gemm fp8_mqa_logits
    (vllm_metax/utils/deep_gemm.py:306-349)."""
    s = torch.einsum("mhd,nd->mhn", q.float(), k.float())
    logits = (F.relu(s) * weights.float()[..., None]).sum(dim=1)
    if k_scale is not None:
        logits = logits * k_scale.float()[None, :]
    n = torch.arange(k.shape[0], device=q.device)[None, :]
    mask = (n >= ks[:, None]) & (n < ke[:, None])
    return logits.masked_fill(~mask, float("-inf"))


def top_k_per_row(logits, k: int):
    """Indices of the k largest finite entries per row, -1 padded.  Order is unspecified.
    Ref kernels: sampler.cu:545-569."""
    M, N = logits.shape
    kk = min(k, N)
    vals, idx = torch.topk(logits, kk, dim=-1)
    idx = torch.where(torch.isinf(vals) & (vals < 0), torch.full_like(idx, -1), idx)
    if kk < k:
        idx = F.pad(idx, (0, k - kk), value=-1)
    return idx.to(torch.int32)


def sparse_attn_indexer(q_fp8, weights, idx_cache, block_table, seq_lens, query_start_loc, topk: int,
                        int8: bool = False, bf16: bool = False, return_logits: bool = False):
    """Full indexer: for every new token, top-k cache positions of its own request.

    ``q_fp8 [T,Hi,128]`` (already quantised values as float/fp8), ``weights [T,Hi]`` with the
    q scale folded in.  Returns ``int32 [T, topk]`` per-request positions (-1 pad).
    Semantics: vllm_metax/registry/custom_ops/layers/sparse_attn_indexer/fp8.py:45-393.
    """
    T = q_fp8.shape[0]
    out = torch.full((T, topk), -1, dtype=torch.int32, device=q_fp8.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    all_logits = (torch.full((T, max(sl + [1])), float("-inf"), dtype=torch.float32, device=q_fp8.device)
                  if return_logits else None)
    for b in range(len(sl)):
        s0, s1 = qsl[b], qsl[b + 1]
        if s1 <= s0:
            continue
        if bf16:      # unquantised keys: bf16 [blocks, block_size, 128], no scales
            nblk = (sl[b] + idx_cache.shape[1] - 1) // idx_cache.shape[1]
            kq = idx_cache[block_table[b][:nblk].long()].reshape(-1, idx_cache.shape[-1])[: sl[b]].float()
            sc = torch.ones(sl[b], device=kq.device)
        else:
            kq, sc = gather_indexer_k(idx_cache, block_table[b], sl[b], int8=int8)
        Lq = s1 - s0
        ke = sl[b] - Lq + 1 + torch.arange(Lq, device=q_fp8.device)
        ks = torch.zeros_like(ke)
        lg = mqa_logits(q_fp8[s0:s1], kq, sc, weights[s0:s1], ks, ke)
        out[s0:s1] = top_k_per_row(lg, topk)
        if all_logits is not None:
            all_logits[s0:s1, : lg.shape[1]] = lg
    return (out, all_logits) if return_logits else out


# --------------------------------------------------------------------------- MoE routing
def topk_softmax(gating, topk: int, renormalize: bool, bias: Optional[torch.Tensor] = None):
    """Softmax over experts then top-k.  Returns ``(weights f32 [T,k], ids int32 [T,k])``.
    Ref: moe/topk_softmax_kernels.cu:80-560."""
    p = torch.softmax(gating.float(), dim=-1)
    sel = p if bias is None else p + bias.float()
    _, ids = torch.topk(sel, topk, dim=-1)
    w = p.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True).clamp(min=1e-20)
    return w, ids.to(torch.int32)


def topk_sigmoid(gating, topk: int, renormalize: bool, bias: Optional[torch.Tensor] = None):
    p = torch.sigmoid(gating.float())
    sel = p if bias is None else p + bias.float()
    _, ids = torch.topk(sel, topk, dim=-1)
    w = p.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True).clamp(min=1e-20)
    return w, ids.to(torch.int32)


def topk_softplus_sqrt(gating, topk: int, renormalize: bool, bias=None, routed_scaling_factor: float = 1.0):
    """sqrt(softplus(x)) scores (DeepSeek-V4).  Ref: moe/topk_softplus_sqrt_kernels.cu:90."""
    p = torch.sqrt(F.softplus(gating.float()))
    sel = p if bias is None else p + bias.float()
    _, ids = torch.topk(sel, topk, dim=-1)
    w = p.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True).clamp(min=1e-20)
    return w * routed_scaling_factor, ids.to(torch.int32)


def grouped_topk(gating, topk: int, renormalize: bool, num_expert_group: int, topk_group: int,
                 scoring_func: str = "sigmoid", bias: Optional[torch.Tensor] = None,
                 routed_scaling_factor: float = 1.0):
    """DeepSeek grouped top-k: score -> (+bias) -> per-group top-2 sum (or max without
    bias) -> keep ``topk_group`` groups -> top-k experts -> renorm * scaling.
    Ref: moe/grouped_topk_kernels.cu:547."""
    T, E = gating.shape
    scores = torch.sigmoid(gating.float()) if scoring_func == "sigmoid" else torch.softmax(gating.float(), dim=-1)
    sel = scores if bias is None else scores + bias.float()[None]
    g = sel.reshape(T, num_expert_group, E // num_expert_group)
    gscore = g.topk(2, dim=-1)[0].sum(dim=-1) if bias is not None else g.max(dim=-1)[0]
    gidx = gscore.topk(topk_group, dim=-1)[1]
    gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
    emask = gmask[..., None].expand(T, num_expert_group, E // num_expert_group).reshape(T, E)
    masked = sel.masked_fill(emask == 0, float("-inf"))
    ids = masked.topk(topk, dim=-1)[1]
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True).clamp(min=1e-20)
    return w * routed_scaling_factor, ids.to(torch.int32)


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Sort (token,k) pairs by expert, padding each expert to a multiple of block_size.

    Returns ``(sorted_token_ids [EM], expert_ids [EM/block], num_tokens_post_pad [1])``;
    padding entries hold ``T*topk``.  Ref: moe/moe_align_sum_kernels.cu:326-369.
    """
    flat = topk_ids.reshape(-1).long()
    numel = flat.numel()
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    padded = ((counts + block_size - 1) // block_size) * block_size
    total = int(padded.sum())
    max_pad = numel + num_experts * (block_size - 1)
    max_pad = ((max_pad + block_size - 1) // block_size) * block_size
    sorted_ids = torch.full((max_pad,), numel, dtype=torch.int32, device=topk_ids.device)
    expert_ids = torch.full((max_pad // block_size,), -1, dtype=torch.int32, device=topk_ids.device)
    order = torch.argsort(flat, stable=True)
    starts = torch.cumsum(padded, 0) - padded
    cstarts = torch.cumsum(counts, 0) - counts
    sorted_e = flat[order]
    rank_in_e = torch.arange(numel, device=flat.device) - cstarts[sorted_e]
    sorted_ids[(starts[sorted_e] + rank_in_e)] = order.to(torch.int32)
    blk_e = torch.repeat_interleave(torch.arange(num_experts, device=flat.device), padded // block_size)
    expert_ids[: blk_e.numel()] = blk_e.to(torch.int32)
    return sorted_ids, expert_ids, torch.tensor([total], dtype=torch.int32, device=topk_ids.device)


def moe_sum(x: torch.Tensor) -> torch.Tensor:
    """``[T, topk, H] -> [T, H]``.  Ref: moe_align_sum_kernels.cu:353."""
    return x.float().sum(dim=1).to(x.dtype)


def fused_experts(x, w13, w2, topk_weights, topk_ids, act: str = "silu", *, w13_scale=None, w2_scale=None,
                  block=(128, 128), expert_map: Optional[torch.Tensor] = None, apply_router_weight_on_input=False):
    """Reference MoE: ``sum_k w_k * W2_e( act(W13_e x) )``.

    ``w13 [E, 2I, H]`` (gate | up), ``w2 [E, H, I]``; with ``*_scale`` the weights are
    e4m3 with 128x128 block scales and activations are quantised 1x128 before each GEMM.
    ``expert_map [E_global] -> local id or -1`` restricts to local experts (EP).
    """
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w13.shape[0]
    for e_local in range(E):
        if expert_map is not None:
            e_glob = (expert_map == e_local).nonzero()
            if e_glob.numel() == 0:
                continue
            e_id = int(e_glob[0])
        else:
            e_id = e_local
        sel = (topk_ids == e_id)
        tok, kk = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        wgt = topk_weights[tok, kk].float()[:, None]
        if apply_router_weight_on_input:
            xe = (xe.float() * wgt).to(x.dtype)
        if w13_scale is not None:
            aq, asc = per_token_group_quant_fp8(xe, block[1])
            h = fp8_block_scaled_mm(aq, asc, w13[e_local], w13_scale[e_local], x.dtype, block)
        else:
            h = gemm(xe, w13[e_local])
        h = swigluoai_and_mul(h) if act == "swigluoai" else act_and_mul(h, act)
        if w2_scale is not None:
            aq, asc = per_token_group_quant_fp8(h, block[1])
            y = fp8_block_scaled_mm(aq, asc, w2[e_local], w2_scale[e_local], x.dtype, block)
        else:
            y = gemm(h, w2[e_local])
        y = y.float() if apply_router_weight_on_input else y.float() * wgt
        out.index_add_(0, tok, y)
    return out.to(x.dtype)


# --------------------------------------------------------------------------- sampling
def apply_repetition_penalties(logits, prompt_mask, output_mask, penalties):
    """logit/penalty if >0 else logit*penalty for tokens seen in prompt or output.
    Ref: sampler.cu:14."""
    seen = prompt_mask | output_mask
    p = penalties.float()[:, None]
    lf = logits.float()
    pen = torch.where(lf > 0, lf / p, lf * p)
    return torch.where(seen, pen, lf).to(logits.dtype)


def apply_penalties(logits, output_counts, presence_penalty, frequency_penalty):
    lf = logits.float()
    lf = lf - frequency_penalty.float()[:, None] * output_counts.float()
    lf = lf - presence_penalty.float()[:, None] * (output_counts > 0).float()
    return lf.to(logits.dtype)


def sample(logits, temperature, top_k, top_p, min_p=None, generators=None, uniform: Optional[torch.Tensor] = None):
    """Greedy where temperature==0 else temperature/top-k/top-p/min-p sampling.

    With ``uniform [B]`` in (0,1) sampling is by inverse CDF over the filtered, sorted
    distribution (deterministic given the uniforms - what the CUDA sampler does).
    """
    B, V = logits.shape
    lf = logits.float()
    greedy = lf.argmax(dim=-1)
    t = temperature.float().clamp(min=1e-6)[:, None]
    probs = torch.softmax(lf / t, dim=-1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    cum = torch.cumsum(sp, dim=-1)
    keep = torch.ones_like(sp, dtype=torch.bool)
    if top_k is not None:
        k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k)[:, None]
        keep &= torch.arange(V, device=logits.device)[None, :] < k
    if top_p is not None:
        # upstream's order: top-p is taken over the distribution renormalised to the top-k set
        spk = sp * keep
        spk = spk / spk.sum(dim=-1, keepdim=True)
        keep &= (torch.cumsum(spk, dim=-1) - spk) < top_p.float()[:, None]
    if min_p is not None:
        keep &= sp >= (min_p.float()[:, None] * sp[:, :1])
    keep[:, 0] = True
    sp = sp * keep
    sp = sp / sp.sum(dim=-1, keepdim=True)
    if uniform is not None:
        c = torch.cumsum(sp, dim=-1)
        pos = (c < uniform.float()[:, None]).sum(dim=-1).clamp(max=V - 1)
    else:
        pos = torch.multinomial(sp, 1).squeeze(-1)
    sampled = si.gather(1, pos[:, None]).squeeze(-1)
    return torch.where(temperature <= 0, greedy, sampled)


# --------------------------------------------------------------------------- misc fused
def fused_qk_norm_rope(qkv, num_q, num_k, num_v, head_dim, eps, q_weight, k_weight, cos_sin_cache, is_neox, positions):
    """Per-head RMSNorm on q and k then RoPE, on packed ``qkv [T,(Hq+Hk+Hv)*D]``.
    Ref: fused_qknorm_rope_kernel.cu:104."""
    T = qkv.shape[0]
    q, k, v = qkv.split([num_q * head_dim, num_k * head_dim, num_v * head_dim], dim=-1)
    qn = rms_norm(q.reshape(T, num_q, head_dim), q_weight, eps).reshape(T, -1)
    kn = rms_norm(k.reshape(T, num_k, head_dim), k_weight, eps).reshape(T, -1)
    qr, kr = rotary_embedding(positions, qn, kn, head_dim, cos_sin_cache, is_neox)
    return torch.cat([qr, kr, v], dim=-1)


def permute_cols(a, perm):
    return a[:, perm.long()]


def selective_scan_fwd(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus=False, state=None):
    """Mamba-1 selective scan, ``u/delta [b, d, L]``, ``A [d, n]``, ``B/C [b, n, L]``.
    Returns ``(y [b,d,L], last_state [b,d,n])``.  Ref: mamba/selective_scan_fwd.cu:69."""
    b, d, L = u.shape
    n = A.shape[1]
    dl = delta.float()
    if delta_bias is not None:
        dl = dl + delta_bias.float()[None, :, None]
    if delta_softplus:
        dl = F.softplus(dl)
    h = torch.zeros(b, d, n, dtype=torch.float32, device=u.device) if state is None else state.float().clone()
    ys = []
    for t in range(L):
        dA = torch.exp(dl[:, :, t, None] * A.float()[None])
        dBu = dl[:, :, t, None] * B.float()[:, None, :, t] * u.float()[:, :, t, None]
        h = dA * h + dBu
        ys.append((h * C.float()[:, None, :, t]).sum(-1))
    y = torch.stack(ys, dim=-1)
    if D is not None:
        y = y + u.float() * D.float()[None, :, None]
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(u.dtype), h


def scaled_mm(aq, wq, a_scale, w_scale, out_dtype=torch.bfloat16, azp=None, azp_adj=None, bias=None):
    """fp32 oracle of the W8A8 GEMM (int8 or fp8 operands, per-token / per-channel scales, optional azp)."""
    acc = aq.float() @ wq.float().t()
    if azp_adj is not None:
        adj = azp_adj.float().reshape(1, -1)
        acc = acc - (azp.float().reshape(-1, 1) * adj if azp is not None else adj)
    out = acc * a_scale.float().reshape(-1, 1) * w_scale.float().reshape(1, -1)
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)
