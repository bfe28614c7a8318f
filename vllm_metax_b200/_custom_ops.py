"""Python entry points of every op: CUDA kernels on GPU tensors, PyTorch reference on CPU.

There is exactly one GPU implementation per op (the hand-written sm_100a kernel in
``csrc/``); the PyTorch implementation in ``ops/reference.py`` is the oracle and the
CPU execution path.  On a GPU tensor a missing native library is an error - nothing
falls back silently.

Parity: vllm_metax/_custom_ops.py:55-264 (the ops the reference adds or changes) plus
the upstream ``vllm._custom_ops`` wrappers it relies on for everything else.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional

import torch

from . import envs
from .ops import reference as ref

_LIB = Path(__file__).resolve().parent / "_b200_C.so"
_loaded = False

ACT_CODES = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "fatrelu": 3, "relu2": 4, "mul_silu": 5, "swigluoai": 6,
             "swiglustep": 7, "gelu_new": 8, "gelu_fast": 9, "gelu_quick": 10}
CACHE_KIND = {"same": 0, "fp8_static": 1, "int8_dyn": 2, "fp8_dyn": 3}


def load_native(build_if_missing: bool = True) -> bool:
    """Load ``_b200_C.so`` (building it in-tree when absent and allowed)."""
    global _loaded
    if _loaded:
        return True
    if not _LIB.exists():
        if not build_if_missing or envs.B200_USE_PREBUILT_KERNELS:
            return False
        from ._build import build

        build()
    torch.ops.load_library(str(_LIB))
    _loaded = True
    return True


def native_loaded() -> bool:
    return _loaded


_launches = 0


def launch_count() -> int:
    """Number of native kernel launches issued through this module so far (graph replays are
    accounted by their owners: launches counted during capture x replays)."""
    return _launches


_force_ref = None
_tc_gemm = None


def _use_cuda(t: torch.Tensor) -> bool:
    global _launches, _force_ref
    if not t.is_cuda:
        return False
    if _force_ref is None:
        _force_ref = bool(envs.B200_FORCE_REFERENCE_OPS)
    if _force_ref:
        return False
    if not _loaded and not load_native():
        raise RuntimeError("CUDA tensor given but the native library _b200_C.so is not built; "
                           "run `python -m vllm_metax_b200._build`")
    _launches += 1
    return True


def kernel_status(device: int = 0) -> dict:
    """Read (and clear) the device status word bounded waits and index checks report into."""
    if not _loaded:
        return {"code": 0}
    w = torch.ops.b200.get_status(device)
    vals = w.tolist()
    if vals[0] != 0:
        w.zero_()
    return {"code": vals[0], "where": vals[1], "expected": vals[2], "observed": vals[3]}


def check_kernel_status(device: int = 0) -> None:
    st = kernel_status(device)
    if st["code"] != 0:
        names = {1: "wait timeout", 2: "index out of range", 3: "bad shape"}
        raise RuntimeError(f"kernel reported {names.get(st['code'], st['code'])} at site {st['where']} "
                           f"(expected {st['expected']}, observed {st['observed']})")


# --------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         force_bn: int = 0) -> torch.Tensor:
    """``a [M,K] @ w [N,K]^T (+bias) (+residual)``."""
    if _use_cuda(a) and a.dtype in (torch.bfloat16, torch.float16):
        if out is None:
            out = torch.empty(a.shape[0], w.shape[0], dtype=a.dtype, device=a.device)
        global _tc_gemm
        if _tc_gemm is None:
            _tc_gemm = bool(envs.B200_TCGEN05_GEMM)
        if _tc_gemm:
            if force_bn == 0 and batch_invariant():
                force_bn = 128                 # one tile shape for every token count
            torch.ops.b200.gemm(out, a, w, bias, residual, force_bn, 0)
        else:  # debug switch only: library GEMM
            torch.addmm(bias, a, w.t(), out=out) if bias is not None else torch.mm(a, w.t(), out=out)
            if residual is not None:
                out.add_(residual)
        return out
    y = ref.gemm(a, w, bias)
    if residual is not None:
        y = (y.float() + residual.float()).to(a.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def gemm_silu_mul(a: torch.Tensor, w_interleaved: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated MLP first half in one kernel: ``w_interleaved [2I, K]`` holds (gate_j, up_j) in rows
    (2j, 2j+1); returns ``silu(a @ gate^T) * (a @ up^T)`` of shape ``[M, I]`` - the activation is
    applied in the GEMM epilogue, so the ``[M, 2I]`` intermediate never reaches memory."""
    if _use_cuda(a) and a.dtype in (torch.bfloat16, torch.float16):
        if out is None:
            out = torch.empty(a.shape[0], w_interleaved.shape[0] // 2, dtype=a.dtype, device=a.device)
        torch.ops.b200.gemm(out, a, w_interleaved, bias, None, 128 if batch_invariant() else 0, 1)
        return out
    y = ref.gemm(a, w_interleaved, bias)
    r = (torch.nn.functional.silu(y[:, 0::2].float()) * y[:, 1::2].float()).to(a.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


# --------------------------------------------------------------------------- norms
def rms_norm(x, weight, eps, out=None, gemma: bool = False):
    if _use_cuda(x):
        out = torch.empty_like(x) if out is None else out
        torch.ops.b200.rms_norm(out, x, weight, eps, gemma)
        return out
    y = ref.gemma_rms_norm(x, weight, eps) if gemma else ref.rms_norm(x, weight, eps)
    if out is not None:
        out.copy_(y)
        return out
    return y


def fused_add_rms_norm(x, residual, weight, eps, gemma: bool = False):
    """In place: ``residual += x``; ``x = rmsnorm(residual)``.  Returns ``(x, residual)``."""
    if _use_cuda(x):
        torch.ops.b200.fused_add_rms_norm(x, residual, weight, eps, gemma)
        return x, residual
    r = (x.float() + residual.float()).to(x.dtype)
    y = ref.gemma_rms_norm(r, weight, eps) if gemma else ref.rms_norm(r, weight, eps)
    x.copy_(y)
    residual.copy_(r)
    return x, residual


def head_rms_norm(x, weight, eps, heads: int, head_dim: int):
    """Per-head RMSNorm in place over the first ``heads*head_dim`` columns of ``x [T, *]``."""
    if _use_cuda(x):
        torch.ops.b200.head_rms_norm(x, weight, eps, heads, head_dim)
        return x
    T = x.shape[0]
    v = x[:, : heads * head_dim].reshape(T, heads, head_dim)
    x[:, : heads * head_dim] = ref.rms_norm(v, weight, eps).reshape(T, -1)
    return x


def rms_norm_static_fp8_quant(x, weight, scale, eps, residual=None):
    if _use_cuda(x):
        out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        torch.ops.b200.rms_norm_quant(out, None, scale, x, residual, weight, eps, 0, 0, False, 0.0)
        return out
    if residual is not None:
        y, r = ref.fused_add_rms_norm(x, residual, weight, eps)
        residual.copy_(r)
        return ref.static_scaled_fp8_quant(y, scale)
    return ref.rms_norm_static_fp8_quant(x, weight, scale, eps)


def rms_norm_dynamic_per_token_quant(x, weight, eps, quant_dtype=torch.float8_e4m3fn, residual=None, scale_ub=None):
    if _use_cuda(x):
        out = torch.empty(x.shape, dtype=quant_dtype, device=x.device)
        scales = torch.empty(*x.shape[:-1], 1, dtype=torch.float32, device=x.device)
        torch.ops.b200.rms_norm_quant(out, scales, None, x, residual, weight, eps,
                                      2 if quant_dtype == torch.int8 else 1, 0, False, scale_ub or 0.0)
        return out, scales
    q, s, r = ref.rms_norm_dynamic_per_token_quant(x, weight, eps, quant_dtype, residual, scale_ub)
    if residual is not None:
        residual.copy_(r)
    return q, s


def rms_norm_per_block_quant(x, weight, eps, group_size=128, residual=None, ue8m0=False):
    if _use_cuda(x):
        out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.empty(*x.shape[:-1], x.shape[-1] // group_size, dtype=torch.float32, device=x.device)
        torch.ops.b200.rms_norm_quant(out, scales, None, x, residual, weight, eps, 3, group_size, ue8m0, 0.0)
        return out, scales
    q, s, r = ref.rms_norm_per_block_quant(x, weight, eps, group_size, residual, ue8m0)
    if residual is not None:
        residual.copy_(r)
    return q, s


# --------------------------------------------------------------------------- rope / cache
def _cache_kind(kv_cache, kv_scales) -> int:
    if kv_cache.dtype == torch.int8:
        return CACHE_KIND["int8_dyn"]
    if kv_cache.dtype == torch.float8_e4m3fn:
        return CACHE_KIND["fp8_dyn"] if kv_scales is not None else CACHE_KIND["fp8_static"]
    return CACHE_KIND["same"]


def rotary_embedding(positions, q, k, head_size, cos_sin_cache, is_neox=True, rot_offset=0, inverse=False):
    """In-place RoPE on ``q [T, Hq*D]`` and optionally ``k [T, Hk*D]``."""
    if _use_cuda(q):
        torch.ops.b200.rope_and_cache(positions, q, k, None, cos_sin_cache, head_size, q.shape[-1] // head_size,
                                      0 if k is None else k.shape[-1] // head_size, is_neox, rot_offset, inverse,
                                      None, None, None, 0, 1.0, 1.0)
        return q, k
    qo, ko = ref.rotary_embedding(positions, q, k, head_size, cos_sin_cache, is_neox, rot_offset, inverse)
    q.copy_(qo)
    if k is not None:
        k.copy_(ko)
    return q, k


def reshape_and_cache(key, value, kv_cache, slot_mapping, kv_scales=None, k_scale=1.0, v_scale=1.0):
    """Scatter ``key/value [T, Hkv, D]`` (or ``[T, Hkv*D]``) into the paged cache."""
    if _use_cuda(key):
        D = kv_cache.shape[-1]
        torch.ops.b200.rope_and_cache(None, None, key, value, None, D, 0, kv_cache.shape[3], True, 0, False, kv_cache,
                                      kv_scales, slot_mapping, _cache_kind(kv_cache, kv_scales), k_scale, v_scale)
        return
    H, D = kv_cache.shape[3], kv_cache.shape[4]
    ref.reshape_and_cache(key.reshape(-1, H, D), value.reshape(-1, H, D), kv_cache, slot_mapping, kv_scales, k_scale, v_scale)


def rope_and_cache(positions, q, k, v, head_size, cos_sin_cache, is_neox, kv_cache, slot_mapping, kv_scales=None,
                   k_scale=1.0, v_scale=1.0, rot_offset=0):
    """RoPE on q, k in place and write (k, v) into the paged cache - one kernel on GPU."""
    if _use_cuda(q):
        torch.ops.b200.rope_and_cache(positions, q, k, v, cos_sin_cache, head_size, q.shape[-1] // head_size,
                                      k.shape[-1] // head_size, is_neox, rot_offset, False, kv_cache, kv_scales,
                                      slot_mapping, _cache_kind(kv_cache, kv_scales), k_scale, v_scale)
        return
    rotary_embedding(positions, q, k, head_size, cos_sin_cache, is_neox, rot_offset)
    reshape_and_cache(k, v, kv_cache, slot_mapping, kv_scales, k_scale, v_scale)


def copy_blocks(kv_caches, src_to_dst: torch.Tensor):
    if kv_caches and _use_cuda(kv_caches[0]):
        pairs = src_to_dst.to(torch.int64).contiguous()
        for c in kv_caches:
            torch.ops.b200.copy_blocks(c, pairs)
        return
    ref.copy_blocks(kv_caches, src_to_dst)


def swap_blocks(src, dst, src_to_dst):
    """Block copies between a device cache and a (pinned) host cache; one async copy per block."""
    for s, d in src_to_dst.tolist():
        dst[d].copy_(src[s], non_blocking=True)


def concat_and_cache_mla(kv_c, k_pe, mla_cache, slot_mapping):
    if _use_cuda(kv_c):
        torch.ops.b200.concat_and_cache_mla(kv_c, k_pe, mla_cache, slot_mapping)
        return
    ref.concat_and_cache_mla(kv_c, k_pe, mla_cache, slot_mapping)


def indexer_k_quant_and_cache(k, idx_cache, slot_mapping, block_size: int, ue8m0: bool = False, int8: bool = False):
    """e4m3 keys (V3.2) or int8 keys (V4, ``int8=True``) + one f32 scale per token.
    Parity: vllm_metax/_custom_ops.py:137-149."""
    if _use_cuda(k):
        torch.ops.b200.indexer_k_quant_and_cache(k, idx_cache, slot_mapping, block_size, ue8m0, int8)
        return
    ref.indexer_k_quant_and_cache(k, idx_cache.view(idx_cache.shape[0], -1), slot_mapping, ue8m0=ue8m0, int8=int8)


# --------------------------------------------------------------------------- activations
def act_and_mul(x, act: str = "silu", out=None, p0: float = 0.0, p1: float = 0.0):
    if _use_cuda(x):
        d = x.shape[-1] // 2
        out = torch.empty(*x.shape[:-1], d, dtype=x.dtype, device=x.device) if out is None else out
        if act == "swigluoai":
            p0, p1 = p0 or 1.702, p1 or 7.0
        if act == "swiglustep":
            p1 = p1 or 7.0
        torch.ops.b200.act_and_mul(out, x, ACT_CODES[act], p0, p1)
        return out
    if act == "mul_silu":
        y = ref.mul_and_silu(x)
    elif act == "swigluoai":
        y = ref.swigluoai_and_mul(x, p0 or 1.702, p1 or 7.0)
    elif act == "swiglustep":
        y = ref.swiglustep_and_mul(x, p1 or 7.0)
    elif act == "fatrelu":
        y = ref.act_and_mul(x, act, threshold=p0)
    else:
        y = ref.act_and_mul(x, act)
    if out is not None:
        out.copy_(y)
        return out
    return y


def silu_and_mul(x, out=None):
    return act_and_mul(x, "silu", out)


def activation(x, act: str):
    if _use_cuda(x):
        out = torch.empty_like(x)
        torch.ops.b200.activation(out, x.contiguous(), ACT_CODES[act], 0.0)
        return out
    return ref.activation(x, act)


def silu_and_mul_quant(x, scale):
    if _use_cuda(x):
        out = torch.empty(*x.shape[:-1], x.shape[-1] // 2, dtype=torch.float8_e4m3fn, device=x.device)
        torch.ops.b200.act_and_mul_quant(out, None, scale, x.contiguous(), 0, 0.0, 0.0, 0, False)
        return out
    return ref.silu_and_mul_quant(x, scale)


def silu_and_mul_per_block_quant(x, group_size=128, ue8m0=False, act: str = "silu"):
    if _use_cuda(x):
        d = x.shape[-1] // 2
        out = torch.empty(*x.shape[:-1], d, dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.empty(*x.shape[:-1], d // group_size, dtype=torch.float32, device=x.device)
        torch.ops.b200.act_and_mul_quant(out, scales, None, x.contiguous(), ACT_CODES[act], 0.0, 7.0, group_size, ue8m0)
        return out, scales
    y = ref.swiglustep_and_mul(x) if act == "swiglustep" else ref.silu_and_mul(x)
    return ref.per_token_group_quant_fp8(y, group_size, ue8m0=ue8m0)


# --------------------------------------------------------------------------- attention
_decode_ws: dict = {}


def _decode_workspace(device, numel: int) -> torch.Tensor:
    ws = _decode_ws.get(device)
    if ws is None or ws.numel() < numel:
        ws = torch.empty(max(numel, 1 << 20), dtype=torch.float32, device=device)
        _decode_ws[device] = ws
    return ws


def batch_invariant() -> bool:
    """``B200_BATCH_INVARIANT=1``: see envs.py.  The first call also pins the switches the native GEMM dispatcher reads
    from the environment (it caches them at its first launch)."""
    global _batch_invariant
    if _batch_invariant is None:
        _batch_invariant = bool(envs.B200_BATCH_INVARIANT)
        if _batch_invariant:
            for name in ("B200_GEMM_STREAMK", "B200_GEMM_SPLITK", "B200_GEMM_PAIR", "B200_FUSED_TP_COLLECTIVES",
                         "B200_CASCADE_ATTENTION", "B200_CUSTOM_ALLREDUCE"):
                os.environ[name] = "0"
    return _batch_invariant


_batch_invariant: Optional[bool] = None


def decode_num_splits(batch: int, num_kv_heads: int, max_seq_len: int, row_tiles: int = 1, sms: int = 148) -> int:
    """Enough KV splits to give every SM a CTA, never finer than 256 tokens per split."""
    if batch_invariant():
        return 1                               # the split count follows the batch size: one pass per sequence instead
    ctas = max(1, batch * num_kv_heads * row_tiles)
    if ctas >= sms:
        return 1
    want = (2 * sms + ctas - 1) // ctas
    return max(1, min(want, max(1, max_seq_len // 256), 32))


def paged_attention_decode(q, kv_cache, block_table, seq_lens, scale, *, out=None, kv_scales=None,
                           query_start_loc=None, max_q_len: int = 1, window: int = -1, softcap: float = 0.0,
                           sinks=None, lse_out=None, num_splits: int = 0, max_seq_len: int = 0, k_scale=1.0,
                           v_scale=1.0, causal=True, workspace=None, alibi_slopes=None):
    """Decode attention over the paged cache; ``q [T, Hq, D]``.  ``alibi_slopes [Hq]`` (f32) adds
    ``slope * (kv position - query position)`` to the scores."""
    if _use_cuda(q):
        out = torch.empty(q.shape[0], q.shape[1], kv_cache.shape[-1], dtype=q.dtype, device=q.device) if out is None else out
        B = seq_lens.shape[0]
        Hkv = kv_cache.shape[3]
        if num_splits <= 0:
            g = q.shape[1] // Hkv
            num_splits = decode_num_splits(B, Hkv, max_seq_len or 4096, (max_q_len * g + 15) // 16)
        ws = workspace
        if num_splits > 1 and ws is None:
            ws = _decode_workspace(q.device, num_splits * q.shape[0] * q.shape[1] * (q.shape[2] + 1))
        torch.ops.b200.paged_attention_decode(out, q, kv_cache, kv_scales, block_table, seq_lens, query_start_loc,
                                              scale, window, softcap, sinks, lse_out, ws, num_splits, B, max_q_len,
                                              k_scale, v_scale, causal, alibi_slopes)
        return out
    B = seq_lens.shape[0]
    qsl = query_start_loc if query_start_loc is not None else torch.arange(B + 1, dtype=torch.int32, device=q.device)
    res = ref.paged_attention(q, kv_cache, block_table, seq_lens, qsl, scale, kv_scales=kv_scales, window=window,
                              softcap=softcap, sinks=sinks, k_scale=k_scale, v_scale=v_scale, causal=causal,
                              return_lse=lse_out is not None, alibi_slopes=alibi_slopes)
    if lse_out is not None:
        res, lse = res
        lse_out.copy_(lse)
    if out is not None:
        out.copy_(res)
        return out
    return res


def paged_attention_prefill(q, kv_cache, block_table, seq_lens, query_start_loc, scale, *, out=None, kv_scales=None,
                            max_q_len: int = 0, window: int = -1, softcap: float = 0.0, sinks=None, lse_out=None,
                            k_scale=1.0, v_scale=1.0, causal=True, max_seq_len: int = 0, alibi_slopes=None):
    """Varlen prefill / chunked-prefill attention reading K, V from the paged cache."""
    if _use_cuda(q):
        out = torch.empty(q.shape[0], q.shape[1], kv_cache.shape[-1], dtype=q.dtype, device=q.device) if out is None else out
        B = seq_lens.shape[0]
        D = q.shape[-1]
        if kv_cache.dtype == q.dtype and D in (64, 128) and kv_scales is None:
            torch.ops.b200.attention_prefill(out, q, kv_cache, None, block_table, seq_lens, query_start_loc, None,
                                             scale, window, softcap, sinks, lse_out, B, max_q_len or q.shape[0], causal,
                                             alibi_slopes)
        else:
            # quantised caches / other head sizes: the split-KV kernel handles any query length in 16-row tiles
            paged_attention_decode(q, kv_cache, block_table, seq_lens, scale, out=out, kv_scales=kv_scales,
                                   query_start_loc=query_start_loc, max_q_len=max_q_len or q.shape[0], window=window,
                                   softcap=softcap, sinks=sinks, lse_out=lse_out, num_splits=1, k_scale=k_scale,
                                   v_scale=v_scale, causal=causal, alibi_slopes=alibi_slopes)
        return out
    res = ref.paged_attention(q, kv_cache, block_table, seq_lens, query_start_loc, scale, kv_scales=kv_scales,
                              window=window, softcap=softcap, sinks=sinks, k_scale=k_scale, v_scale=v_scale,
                              causal=causal, return_lse=lse_out is not None, alibi_slopes=alibi_slopes)
    if lse_out is not None:
        res, lse = res
        lse_out.copy_(lse)
    if out is not None:
        out.copy_(res)
        return out
    return res


def varlen_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, scale, *, out=None, max_q_len: int = 0, causal=True,
                     window: int = -1, softcap: float = 0.0, sinks=None, lse_out=None):
    """Ragged attention over contiguous ``k [Tk,Hkv,Dqk]``, ``v [Tk,Hkv,Dv]`` (MLA prefill, ViT)."""
    if _use_cuda(q):
        out = torch.empty(q.shape[0], q.shape[1], v.shape[-1], dtype=q.dtype, device=q.device) if out is None else out
        B = cu_seqlens_q.shape[0] - 1
        torch.ops.b200.attention_prefill(out, q, k, v, None, None, cu_seqlens_q, cu_seqlens_k, scale, window, softcap,
                                         sinks, lse_out, B, max_q_len or q.shape[0], causal)
        return out
    T, Hq, _ = q.shape
    res = torch.zeros(T, Hq, v.shape[-1], dtype=torch.float32, device=q.device)
    lse_all = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for b in range(len(cq) - 1):
        if cq[b + 1] <= cq[b]:
            continue
        lq, lk = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        o, lse = ref.attention_core(q[cq[b]:cq[b + 1]].float(), k[ck[b]:ck[b + 1]].float(), v[ck[b]:ck[b + 1]].float(),
                                    scale, causal_offset=(lk - lq) if causal else None, window=window,
                                    softcap=softcap, sinks=sinks)
        res[cq[b]:cq[b + 1]] = o
        lse_all[:, cq[b]:cq[b + 1]] = lse
    if lse_out is not None:
        lse_out.copy_(lse_all)
    res = res.to(q.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


# --------------------------------------------------------------------------- sampling
def argmax(logits, out=None):
    if _use_cuda(logits):
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device) if out is None else out
        torch.ops.b200.argmax(out, logits)
        return out
    r = logits.float().argmax(dim=-1)
    if out is not None:
        out.copy_(r)
        return out
    return r


def sample(logits, temperature, top_k=None, top_p=None, min_p=None, uniform=None, out=None):
    if _use_cuda(logits):
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device) if out is None else out
        if uniform is None:
            uniform = torch.rand(logits.shape[0], dtype=torch.float32, device=logits.device)
        torch.ops.b200.sample(out, logits, temperature, top_k, top_p, min_p, uniform)
        return out
    r = ref.sample(logits, temperature, top_k, top_p, min_p, uniform=uniform)
    if out is not None:
        out.copy_(r)
        return out
    return r


def apply_penalties(logits, prompt_mask, output_counts, rep, presence, frequency):
    """In place.  ``prompt_mask``/``output_counts`` are int32 ``[B, V]``.  Parity: csrc/sampler.cu:14."""
    if _use_cuda(logits):
        torch.ops.b200.apply_penalties(logits, prompt_mask, output_counts, rep, presence, frequency)
        return logits
    lf = logits
    if rep is not None:
        pm = prompt_mask.bool() if prompt_mask is not None else torch.zeros_like(logits, dtype=torch.bool)
        om = output_counts > 0 if output_counts is not None else torch.zeros_like(logits, dtype=torch.bool)
        lf = ref.apply_repetition_penalties(lf, pm, om, rep)
    if output_counts is not None and (presence is not None or frequency is not None):
        z = torch.zeros(logits.shape[0], device=logits.device)
        lf = ref.apply_penalties(lf, output_counts, presence if presence is not None else z,
                                 frequency if frequency is not None else z)
    logits.copy_(lf)
    return logits


def advance_step(input_ids, positions, seq_lens, slot_mapping, sampled, block_table, block_size, batch,
                 token_log=None, log_col: int = 0):
    if _use_cuda(input_ids):
        torch.ops.b200.advance_step(input_ids, positions, seq_lens, slot_mapping, sampled, block_table, block_size,
                                    batch, token_log, log_col)
        return
    input_ids[:batch] = sampled[:batch]
    if token_log is not None:
        token_log[:batch, log_col] = sampled[:batch]
    positions[:batch] += 1
    seq_lens[:batch] = (positions[:batch] + 1).to(seq_lens.dtype)
    pos = positions[:batch]
    blk = block_table[torch.arange(batch), (pos // block_size).long()].long()
    slot_mapping[:batch] = blk * block_size + pos % block_size


def embedding(table, ids, out=None, vocab_start: int = 0):
    if _use_cuda(table) and table.dtype in (torch.bfloat16, torch.float16):
        out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device) if out is None else out
        torch.ops.b200.embedding(out, table, ids, vocab_start)
        return out
    local = ids - vocab_start
    ok = (local >= 0) & (local < table.shape[0])
    y = table[local.clamp(0, table.shape[0] - 1)] * ok[:, None].to(table.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


# --------------------------------------------------------------------------- MoE routing / shuffling
_GATING_MODE = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def topk_gating(gating, topk: int, renormalize: bool, scoring: str = "softmax", bias=None, scale: float = 1.0):
    """Fused score + top-k (+ renorm, scale).  Returns ``(weights f32 [T,k], ids int32 [T,k])``.
    Parity: torch.ops._moe_C.topk_softmax / topk_sigmoid / topk_softplus_sqrt."""
    if _use_cuda(gating):
        T = gating.shape[0]
        w = torch.empty(T, topk, dtype=torch.float32, device=gating.device)
        ids = torch.empty(T, topk, dtype=torch.int32, device=gating.device)
        torch.ops.b200.topk_gating(w, ids, gating.contiguous(), bias, _GATING_MODE[scoring], renormalize, scale)
        return w, ids
    if scoring == "softmax":
        w, ids = ref.topk_softmax(gating, topk, renormalize, bias)
    elif scoring == "sigmoid":
        w, ids = ref.topk_sigmoid(gating, topk, renormalize, bias)
    else:
        return ref.topk_softplus_sqrt(gating, topk, renormalize, bias, scale)
    return w * scale, ids


def grouped_topk(gating, topk: int, renormalize: bool, num_expert_group: int, topk_group: int,
                 scoring_func: str = "sigmoid", bias=None, routed_scaling_factor: float = 1.0):
    """Parity: vllm_metax/_custom_ops.py:206-238 (grouped_topk).  ``B200_USE_FUSED_GROUPED_TOPK=0`` takes the unfused
    PyTorch statement on the device instead of the kernel (the reference's ``MACA_VLLM_USE_FUSED_GROUPED_TOPK``-style
    switch for bisecting routing differences)."""
    if _use_cuda(gating) and envs.B200_USE_FUSED_GROUPED_TOPK:
        T = gating.shape[0]
        w = torch.empty(T, topk, dtype=torch.float32, device=gating.device)
        ids = torch.empty(T, topk, dtype=torch.int32, device=gating.device)
        torch.ops.b200.grouped_topk(w, ids, gating.contiguous(), None if bias is None else bias.float(),
                                    num_expert_group, topk_group, scoring_func == "sigmoid", renormalize,
                                    routed_scaling_factor)
        return w, ids
    return ref.grouped_topk(gating, topk, renormalize, num_expert_group, topk_group, scoring_func, bias,
                            routed_scaling_factor)


def moe_align_block_size(topk_ids, block_size: int, num_experts: int, expert_map=None, want_inverse: bool = False):
    """Expert-sort (token, k) pairs with per-expert padding to ``block_size``.

    Returns ``(sorted_token_ids, block_expert_ids, num_tokens_post_padded[, inverse positions])``; padding
    entries of ``sorted_token_ids`` hold ``numel``.  With ``expert_map`` (global -> local id or -1) pairs
    routed to other ranks are dropped (their inverse position is -1)."""
    numel = topk_ids.numel()
    max_pad = numel + num_experts * (block_size - 1)
    max_pad = (max_pad + block_size - 1) // block_size * block_size
    if _use_cuda(topk_ids):
        dev = topk_ids.device
        sorted_ids = torch.empty(max_pad, dtype=torch.int32, device=dev)
        block_expert = torch.empty(max_pad // block_size, dtype=torch.int32, device=dev)
        total = torch.empty(1, dtype=torch.int32, device=dev)
        inv = torch.empty(numel, dtype=torch.int32, device=dev) if want_inverse else None
        torch.ops.b200.moe_align(sorted_ids, block_expert, total, inv, topk_ids.contiguous(), expert_map, num_experts,
                                 block_size)
        return (sorted_ids, block_expert, total, inv) if want_inverse else (sorted_ids, block_expert, total)
    ids = topk_ids.reshape(-1).long()
    if expert_map is not None:
        ids = expert_map.long()[ids]
    keep = ids >= 0
    flat = torch.where(keep, ids, torch.full_like(ids, num_experts))
    counts = torch.bincount(flat, minlength=num_experts + 1)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    starts = torch.cumsum(padded, 0) - padded
    sorted_ids = torch.full((max_pad,), numel, dtype=torch.int32)
    block_expert = torch.full((max_pad // block_size,), -1, dtype=torch.int32)
    inv = torch.full((numel,), -1, dtype=torch.int32)
    order = torch.argsort(flat, stable=True)
    order = order[flat[order] < num_experts]
    se = flat[order]
    cstarts = torch.cumsum(counts, 0) - counts
    pos = starts[se] + (torch.arange(order.numel()) - cstarts[se])
    sorted_ids[pos] = order.to(torch.int32)
    inv[order] = pos.to(torch.int32)
    be = torch.repeat_interleave(torch.arange(num_experts), padded // block_size)
    block_expert[: be.numel()] = be.to(torch.int32)
    total = padded.sum().to(torch.int32).reshape(1)
    return (sorted_ids, block_expert, total, inv) if want_inverse else (sorted_ids, block_expert, total)


def moe_gather(x, sorted_ids, total_padded, topk: int):
    """Rows of ``x [T,H]`` in expert-sorted order, zero rows for padding: ``[max_padded, H]``."""
    if _use_cuda(x):
        out = torch.empty(sorted_ids.numel(), x.shape[1], dtype=x.dtype, device=x.device)
        torch.ops.b200.moe_gather(out, x.contiguous(), sorted_ids, total_padded, topk)
        return out
    numel = x.shape[0] * topk
    sid = sorted_ids.long()
    valid = sid < numel
    out = torch.zeros(sid.numel(), x.shape[1], dtype=x.dtype)
    out[valid] = x[sid[valid] // topk]
    return out


def gemm_grouped(a, w, block_expert, total_padded, epi: int = 0):
    """Per-row-block expert GEMM: ``a [R, K]`` (R multiple of 128), ``w [E, N, K]`` -> ``[R, N]`` (``N/2`` with the
    SiLU-gate epilogue over row-interleaved gate/up weights)."""
    if _use_cuda(a):
        n_out = w.shape[1] // 2 if epi == 1 else w.shape[1]
        out = torch.empty(a.shape[0], n_out, dtype=a.dtype, device=a.device)
        torch.ops.b200.gemm_grouped(out, a, w, block_expert, total_padded, epi)
        return out
    R = a.shape[0]
    nblk = R // 128
    n_out = w.shape[1] // 2 if epi == 1 else w.shape[1]
    out = torch.zeros(R, n_out, dtype=a.dtype)
    valid_blocks = int(total_padded.item()) // 128
    for b in range(min(nblk, valid_blocks)):
        e = int(block_expert[b])
        if e < 0:
            continue
        y = ref.gemm(a[b * 128:(b + 1) * 128], w[e])
        if epi == 1:
            y = (torch.nn.functional.silu(y[:, 0::2].float()) * y[:, 1::2].float()).to(a.dtype)
        out[b * 128:(b + 1) * 128] = y
    return out


def moe_combine(y, weights, inv_pos, tokens: int, shared=None):
    """``out[t] = sum_k weights[t,k] * y[inv_pos[t,k]] (+ shared[t])``."""
    if _use_cuda(y):
        out = torch.empty(tokens, y.shape[1], dtype=y.dtype, device=y.device)
        torch.ops.b200.moe_combine(out, y, weights.contiguous(), inv_pos, shared)
        return out
    topk = weights.shape[1]
    ip = inv_pos.reshape(tokens, topk).long()
    ok = ip >= 0
    g = y[ip.clamp(min=0)].float() * (weights.float() * ok)[..., None]
    out = g.sum(dim=1)
    if shared is not None:
        out = out + shared.float()
    return out.to(y.dtype)


def moe_sum(x):
    if _use_cuda(x):
        out = torch.empty(x.shape[0], x.shape[2], dtype=x.dtype, device=x.device)
        torch.ops.b200.moe_sum(out, x.contiguous())
        return out
    return ref.moe_sum(x)


# --------------------------------------------------------------------------- quantisation
def per_token_group_quant_fp8(x, group_size: int = 128, ue8m0: bool = False, column_major_scales: bool = False,
                              eps: float = 1e-10):
    """1 x group dynamic e4m3 quantisation: ``(q, scales [.., K/g])`` (scales ``[K/g, rows]`` if column-major)."""
    if _use_cuda(x):
        xc = x.contiguous()
        K = xc.shape[-1]
        rows = xc.numel() // K
        q = torch.empty(xc.shape, dtype=torch.float8_e4m3fn, device=x.device)
        shape = (K // group_size, rows) if column_major_scales else (*xc.shape[:-1], K // group_size)
        s = torch.empty(shape, dtype=torch.float32, device=x.device)
        torch.ops.b200.per_token_group_quant(q, s, xc, group_size, ue8m0, column_major_scales, eps)
        return q, s
    q, s = ref.per_token_group_quant_fp8(x, group_size, eps, ue8m0)
    return (q, s.reshape(-1, s.shape[-1]).t().contiguous()) if column_major_scales else (q, s)


def per_token_group_quant_int8(x, group_size: int = 128, eps: float = 1e-10):
    if _use_cuda(x):
        xc = x.contiguous()
        q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
        s = torch.empty(*xc.shape[:-1], xc.shape[-1] // group_size, dtype=torch.float32, device=x.device)
        torch.ops.b200.per_token_group_quant(q, s, xc, group_size, False, False, eps)
        return q, s
    return ref.per_token_group_quant_int8(x, group_size, eps)


def scaled_fp8_quant(x, scale=None, use_per_token_if_dynamic: bool = False, scale_ub=None):
    """Static (``scale`` given), dynamic per-tensor, or dynamic per-token fp8 quantisation."""
    if _use_cuda(x):
        xc = x.contiguous()
        q = torch.empty(xc.shape, dtype=torch.float8_e4m3fn, device=x.device)
        if scale is not None:
            torch.ops.b200.scaled_fp8_quant(q, scale, xc, 0, 0.0)
            return q, scale
        if use_per_token_if_dynamic:
            s = torch.empty(*xc.shape[:-1], 1, dtype=torch.float32, device=x.device)
            torch.ops.b200.scaled_fp8_quant(q, s, xc, 1, scale_ub or 0.0)
            return q, s
        s = (xc.abs().max().float() / 448.0).clamp(min=1e-12).reshape(1)
        torch.ops.b200.scaled_fp8_quant(q, s, xc, 0, 0.0)
        return q, s
    if scale is not None:
        return ref.static_scaled_fp8_quant(x, scale), scale
    if use_per_token_if_dynamic:
        return ref.dynamic_per_token_scaled_fp8_quant(x, scale_ub)
    return ref.dynamic_scaled_fp8_quant(x)


def scaled_int8_quant(x, scale=None, azp=None, symmetric: bool = True):
    """Returns ``(q, scale, azp_or_None)``.  Parity: vllm_metax patch utils._int8_quantize -> scaled_int8_quant."""
    if _use_cuda(x):
        xc = x.contiguous()
        q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
        if scale is not None:
            torch.ops.b200.scaled_int8_quant(q, scale, azp, xc, 0 if symmetric else 1)
            return q, scale, azp
        s = torch.empty(*xc.shape[:-1], 1, dtype=torch.float32, device=x.device)
        z = None if symmetric else torch.empty(*xc.shape[:-1], 1, dtype=torch.int32, device=x.device)
        torch.ops.b200.scaled_int8_quant(q, s, z, xc, 2 if symmetric else 3)
        return q, s, z
    return ref.scaled_int8_quant(x, scale, azp, symmetric)


def merge_attn_states(prefix_out, prefix_lse, suffix_out, suffix_lse, want_lse: bool = False):
    if _use_cuda(prefix_out):
        prefix_out, prefix_lse = prefix_out.contiguous(), prefix_lse.contiguous()     # (empty_like keeps odd strides)
        out = torch.empty_like(prefix_out)
        lse = torch.empty_like(prefix_lse) if want_lse else None
        torch.ops.b200.merge_attn_states(out, lse, prefix_out, prefix_lse,
                                         suffix_out.contiguous(), suffix_lse.contiguous())
        return (out, lse) if want_lse else out
    out, lse = ref.merge_attn_states(prefix_out, prefix_lse, suffix_out, suffix_lse)
    return (out, lse) if want_lse else out


def fp8_block_scaled_mm(aq, a_scale, wq, w_scale, out_dtype=torch.bfloat16, block_expert=None, total_padded=None):
    """Block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales); grouped when ``wq`` is 3-D."""
    if _use_cuda(aq):
        n = wq.shape[-2]
        out = torch.empty(aq.shape[0], n, dtype=out_dtype, device=aq.device)
        torch.ops.b200.gemm_fp8_blockscale(out, aq, a_scale.contiguous(), wq, w_scale.contiguous(), block_expert,
                                           total_padded)
        return out
    if wq.dim() == 2:
        return ref.fp8_block_scaled_mm(aq, a_scale, wq, w_scale, out_dtype)
    out = torch.zeros(aq.shape[0], wq.shape[1], dtype=out_dtype)
    for b in range(int(total_padded.item()) // 128):
        e = int(block_expert[b])
        if e >= 0:
            sl = slice(b * 128, (b + 1) * 128)
            out[sl] = ref.fp8_block_scaled_mm(aq[sl], a_scale[sl], wq[e], w_scale[e], out_dtype)
    return out


def scaled_mm(aq, wq, a_scale, w_scale, out_dtype=torch.bfloat16, *, azp=None, azp_adj=None, bias=None,
              block_expert=None, total_padded=None):
    """W8A8 GEMM ``out = a_scale * w_scale * (aq @ wq.T - azp * azp_adj) + bias``.

    ``aq [M,K]`` and ``wq [N,K]`` (or ``[E,N,K]`` grouped over expert-sorted rows) are int8 or fp8 e4m3;
    ``a_scale`` has 1 or M entries, ``w_scale`` 1 or N per expert.  ``azp_adj [N]`` int32 = column sums of
    ``wq`` (times the zero point when that is per tensor, in which case ``azp`` is None); ``azp [M]`` int32 is
    the per-token zero point.  Parity: cutlass_scaled_mm / cutlass_scaled_mm_azp / cutlass_moe_mm_w8a8,
    vllm_metax/model_executor/layers/quantization/_python_api_ops.py:812-1105."""
    if _use_cuda(aq):
        out = torch.empty(aq.shape[0], wq.shape[-2], dtype=out_dtype, device=aq.device)
        torch.ops.b200.scaled_mm(out, aq, wq, a_scale.float().reshape(-1).contiguous(),
                                 w_scale.float().reshape(-1).contiguous(),
                                 None if azp is None else azp.int().reshape(-1).contiguous(),
                                 None if azp_adj is None else azp_adj.int().reshape(-1).contiguous(),
                                 bias, block_expert, total_padded)
        return out
    if wq.dim() == 2:
        return ref.scaled_mm(aq, wq, a_scale, w_scale, out_dtype, azp, azp_adj, bias)
    out = torch.zeros(aq.shape[0], wq.shape[1], dtype=out_dtype)
    ws = w_scale.float().reshape(wq.shape[0], -1)
    for b in range(int(total_padded.item()) // 128):
        e = int(block_expert[b])
        if e >= 0:
            sl = slice(b * 128, (b + 1) * 128)
            asl = a_scale.reshape(-1)[sl] if a_scale.numel() > 1 else a_scale
            out[sl] = ref.scaled_mm(aq[sl], wq[e], asl, ws[e], out_dtype)
    return out


def wna16_token_tile(rows_per_expert: int) -> int:
    """Token tile (= moe_align block size) the weight-only GEMM uses for about this many rows per expert."""
    m = max(int(rows_per_expert), 1)
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def wna16_gemm(x, qweight, scales, zeros, bits: int, group: int, *, bias=None, block_expert=None, total_padded=None,
               token_tile: int = 0, silu_gate: bool = False):
    """``x [M,K] @ dequant(qweight)^T`` with 4/8-bit group-quantised weights in the canonical layout
    (``quantization/wna16.py``); grouped over expert-sorted rows when ``qweight`` is 3-D.  ``silu_gate``
    applies SiLU(gate) * up over interleaved output rows (output width N/2)."""
    N = qweight.shape[-2]
    if _use_cuda(x):
        out = torch.empty(x.shape[0], N // 2 if silu_gate else N, dtype=x.dtype, device=x.device)
        torch.ops.b200.wna16_gemm(out, x, qweight, scales, zeros, bits, group, bias, block_expert, total_padded,
                                  token_tile, 1 if silu_gate else 0)
        return out
    from .quantization.wna16 import dequantize_canonical

    def one(xs, q, s, z):
        y = xs.float() @ dequantize_canonical(q, s, z, bits, group).to(x.dtype).float().t()
        if bias is not None:
            y = y + bias.float()
        if silu_gate:
            y = y.to(x.dtype).float()
            y = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
        return y.to(x.dtype)

    if qweight.dim() == 2:
        return one(x, qweight, scales, zeros)
    out = torch.zeros(x.shape[0], N // 2 if silu_gate else N, dtype=x.dtype)
    for b in range(int(total_padded.item()) // token_tile):
        e = int(block_expert[b])
        if e >= 0:
            sl = slice(b * token_tile, (b + 1) * token_tile)
            out[sl] = one(x[sl], qweight[e], scales[e], zeros[e])
    return out


# --------------------------------------------------------------------------- MLA
def mla_decode(q, mla_cache, block_table, seq_lens, scale, *, query_start_loc=None, topk_indices=None, out=None,
               lse_out=None, num_splits: int = 0, max_seq_len: int = 0, impl: int = 0):
    """Absorbed MLA over the latent cache (dense, or sparse with ``topk_indices [T, topk]``).
    ``q [T, H, 576]`` -> ``[T, H, 512]``.  ``impl``: 0 = choose, 1 = mma.sync kernel, 2 = tcgen05 kernel (dense 16-bit
    caches; csrc/mla_decode_tcgen05.cu) or fail.  "Choose" takes the tcgen05 kernel for 64 heads per rank or more only
    with ``B200_MLA_TCGEN05=1``."""
    if _use_cuda(q):
        T, H, _ = q.shape
        if impl == 0 and not envs.B200_MLA_TCGEN05:
            impl = 1
        out = torch.empty(T, H, 512, dtype=q.dtype, device=q.device) if out is None else out
        if num_splits <= 0 and batch_invariant():
            num_splits = 1
        if num_splits <= 0:
            # heads per CTA as chosen by the kernel launcher (csrc/mla_decode.cu:mla_decode_heads_per_cta)
            hpc = 16 if H <= 16 else (32 if (H <= 32 or mla_cache.dtype == torch.uint8) else 64)
            ctas = T * ((H + hpc - 1) // hpc)
            if impl != 1 and topk_indices is None and mla_cache.dtype != torch.uint8 and (impl == 2 or H >= 64):
                ctas = 2 * T * ((H + 127) // 128)            # tcgen05 kernel: 128 heads x half the latent per CTA
            kv = topk_indices.shape[1] if topk_indices is not None else (max_seq_len or 4096)
            num_splits = 1 if ctas >= 148 else max(1, min((296 + ctas - 1) // ctas, kv // 256, 16))
        ws = _decode_workspace(q.device, num_splits * T * H * 513) if num_splits > 1 else None
        torch.ops.b200.mla_decode(out, q, mla_cache, block_table, seq_lens, query_start_loc, topk_indices, scale,
                                  lse_out, ws, num_splits, impl)
        return out
    res, lse = ref.mla_decode(q, mla_cache, block_table, seq_lens, scale, query_start_loc=query_start_loc,
                              topk_indices=topk_indices)
    if lse_out is not None:
        lse_out.copy_(lse)
    if out is not None:
        out.copy_(res)
        return out
    return res


# --------------------------------------------------------------------------- DSA indexer
def top_k_per_row(logits, k: int, row_len=None):
    """Indices of the k largest finite entries per row (-1 padded, unordered).
    Parity: vllm_metax/_custom_ops.py:170-203 (top_k_per_row / top_k_per_row_decode)."""
    if _use_cuda(logits):
        out = torch.empty(logits.shape[0], k, dtype=torch.int32, device=logits.device)
        torch.ops.b200.topk_per_row(out, logits, row_len, logits.shape[1])
        return out
    if row_len is not None:
        n = torch.arange(logits.shape[1])[None, :]
        logits = logits.masked_fill(n >= row_len[:, None], float("-inf"))
    return ref.top_k_per_row(logits, k)


def indexer_topk(q_fp8, weights, idx_cache, block_table, seq_lens, query_start_loc, topk: int, block_size: int,
                 max_seq_len: int = 0, return_logits: bool = False, max_query_len: int = 0, impl: int = 0):
    """Index logits of every new token against its request's cached keys, then top-k.  ``q_fp8`` is e4m3, or int8
    (the V4 indexer: queries from ``ops.v4_cache.indexer_q_rope_int8_quant``, keys written with ``int8=True``).
    Returns int32 ``[T, topk]`` per-request positions (-1 = none)."""
    if _use_cuda(q_fp8):
        T = q_fp8.shape[0]
        L = max(int(max_seq_len), 1)
        Lp = (L + 1023) // 1024 * 1024
        logits = torch.empty(T, Lp, dtype=torch.float32, device=q_fp8.device)
        i8 = q_fp8.dtype == torch.int8
        if q_fp8.dtype == torch.bfloat16:        # unquantised indexer: ``idx_cache`` is bf16 [blocks, block_size, 128]
            qb = q_fp8
            idx_cache = idx_cache.view(torch.uint8).reshape(idx_cache.shape[0], -1)
        else:
            qb = q_fp8 if (i8 or q_fp8.dtype == torch.float8_e4m3fn) else q_fp8.to(torch.float8_e4m3fn)
        torch.ops.b200.indexer_logits(logits, qb.contiguous(), weights.float().contiguous(), idx_cache, block_table,
                                      seq_lens, query_start_loc, block_size, L, i8, int(max_query_len), int(impl))
        _ = _use_cuda(q_fp8)  # second kernel of the op (launch accounting)
        out = torch.empty(T, topk, dtype=torch.int32, device=q_fp8.device)
        torch.ops.b200.topk_per_row(out, logits, None, Lp)
        return (out, logits) if return_logits else out
    return ref.sparse_attn_indexer(q_fp8.float(), weights, idx_cache, block_table, seq_lens, query_start_loc, topk,
                                   int8=q_fp8.dtype == torch.int8, bf16=q_fp8.dtype == torch.bfloat16,
                                   return_logits=return_logits)
