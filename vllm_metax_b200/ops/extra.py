"""Wrappers of the small fused kernels (min-latency GEMM, fused q/k norm + RoPE, MLA RoPE + cache insert,
cache gathers, column permute, Mamba selective scan).  CUDA tensors run the kernels of
``csrc/small_gemm.cu``, ``csrc/fused_misc.cu`` and ``csrc/mamba_scan.cu``; CPU tensors run the fp32
PyTorch statement of the same op, which is also the oracle the kernels are tested against.

Parity: vllm_metax/_custom_ops.py (``dsv3_fused_a_gemm``, ``router_gemm_*``, ``fused_qk_norm_rope``,
``concat_and_cache_mla_rope_fused``, ``concat_mla_q``, ``permute_cols``, ``gather_and_maybe_dequant_cache``,
``cp_gather_indexer_k_quant_cache``, ``selective_scan_fwd``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _custom_ops as ops
from . import reference as ref


def _cuda(x: torch.Tensor) -> bool:
    return ops._use_cuda(x)


def small_gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M<=32, K] @ w [N, K]^T`` with the cluster split-K tensor-core kernel; ``out_dtype=torch.float32``
    gives fp32 logits (router GEMM).  Larger M falls back to the general GEMM."""
    out_dtype = out_dtype or x.dtype
    if _cuda(x) and x.shape[0] <= 32 and x.shape[1] % 32 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1:
        out = torch.empty(x.shape[0], w.shape[0], dtype=out_dtype, device=x.device)
        torch.ops.b200.small_gemm(out, x, w, bias)
        return out
    if _cuda(x):
        return ops.gemm(x, w, bias).to(out_dtype)
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def router_gemm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """MoE router logits in fp32."""
    return small_gemm(x, w, None, torch.float32)


def fused_qk_norm_rope(qkv: torch.Tensor, q_weight, k_weight, cos_sin_cache, positions, num_q: int, num_k: int,
                       num_v: int, head_dim: int, is_neox: bool = True, eps: float = 1e-6, gemma: bool = False):
    """In place on packed ``qkv [T, (Hq+Hk+Hv)*D]``: per-head RMSNorm of q and k, then RoPE over the first
    ``cos_sin_cache.shape[1]`` dims of every q / k head."""
    if _cuda(qkv):
        torch.ops.b200.fused_qk_norm_rope(qkv, q_weight, k_weight, cos_sin_cache, positions, num_q, num_k, num_v,
                                          head_dim, is_neox, eps, gemma)
        return qkv
    T = qkv.shape[0]
    D = head_dim
    q = qkv[:, : num_q * D].reshape(T, num_q, D)
    k = qkv[:, num_q * D: (num_q + num_k) * D].reshape(T, num_k, D)
    norm = ref.gemma_rms_norm if gemma else ref.rms_norm
    qn = norm(q, q_weight, eps).reshape(T, -1)
    kn = norm(k, k_weight, eps).reshape(T, -1)
    qo, ko = ref.rotary_embedding(positions, qn, kn, D, cos_sin_cache, is_neox)
    qkv[:, : num_q * D] = qo
    qkv[:, num_q * D: (num_q + num_k) * D] = ko
    return qkv


def qkv_norm_rope_insert(qkv: torch.Tensor, positions, slot_mapping, cos_sin_cache, num_q: int, num_kv: int,
                         q_weight=None, k_weight=None, kv_cache=None, num_index_q: int = 0, index_k: bool = False,
                         index_q_weight=None, index_k_weight=None, index_cache=None, index_fp8: bool = False,
                         is_neox: bool = True, eps: float = 1e-6, gemma: bool = True):
    """One pass over ``qkv [T, (Hq + 2 Hkv + Niq + index_k) * 128]`` (MiniMax-M3 layout): per-head (gemma) RMSNorm +
    partial RoPE of q, k, index_q, index_k; ``q`` / ``index_q`` are returned as contiguous ``[T, H, 128]``; k (also
    rewritten in place) and v go into ``kv_cache [blocks, 2, block_size, Hkv, 128]``, index_k into
    ``index_cache [slots, 128]`` at ``slot_mapping`` (shorter than T: the tail gets no cache rows; negative slots are
    skipped).  ``index_fp8`` stores index_q / index_k as e4m3 bytes (direct saturating cast).
    Returns ``(q_out, index_q_out or None)``."""
    T, D = qkv.shape[0], 128
    if _cuda(qkv):
        q_out = torch.empty(T, num_q, D, dtype=qkv.dtype, device=qkv.device)
        iq_out = None
        if num_index_q:
            iq_out = torch.empty(T, num_index_q, D, dtype=torch.uint8 if index_fp8 else qkv.dtype, device=qkv.device)
        torch.ops.b200.qkv_norm_rope_insert(qkv, q_out, iq_out, kv_cache, index_cache if index_k else None, q_weight,
                                            k_weight, index_q_weight, index_k_weight, cos_sin_cache,
                                            positions.long().contiguous(), slot_mapping.long().contiguous(), num_q,
                                            num_kv, num_index_q, index_k, is_neox, eps, gemma)
        return q_out, iq_out
    norm = ref.gemma_rms_norm if gemma else ref.rms_norm

    def nr(x, w):                                    # x [T, h, 128]
        h = x.shape[1]
        y = norm(x, w, eps) if w is not None else x
        y, _ = ref.rotary_embedding(positions[:T], y.reshape(T, h * D), None, D, cos_sin_cache, is_neox)
        return y.reshape(T, h, D)

    def fp8(x):
        return x.float().clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)

    o = 0
    q = qkv[:, o: o + num_q * D].reshape(T, num_q, D); o += num_q * D
    k = qkv[:, o: o + num_kv * D].reshape(T, num_kv, D); ko = o; o += num_kv * D
    v = qkv[:, o: o + num_kv * D].reshape(T, num_kv, D); o += num_kv * D
    q_out = nr(q, q_weight).contiguous()
    k_out = nr(k, k_weight)
    qkv[:, ko: ko + num_kv * D] = k_out.reshape(T, -1)
    iq_out = ik_out = None
    if num_index_q:
        iq = nr(qkv[:, o: o + num_index_q * D].reshape(T, num_index_q, D), index_q_weight)
        iq_out = fp8(iq) if index_fp8 else iq.contiguous()
        o += num_index_q * D
    if index_k:
        ik_out = nr(qkv[:, o: o + D].reshape(T, 1, D), index_k_weight)[:, 0]
    n = slot_mapping.numel()
    for t in range(n):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        if kv_cache is not None:
            blk, pos = divmod(s, kv_cache.shape[2])
            kv_cache[blk, 0, pos] = k_out[t]
            kv_cache[blk, 1, pos] = v[t]
        if index_k and index_cache is not None:
            index_cache.view(-1, D)[s] = fp8(ik_out[t]) if index_fp8 else ik_out[t]
    return q_out, iq_out


def mla_rope_and_cache(q_pe, k_pe, kv_c, mla_cache, cos_sin_cache, positions, slot_mapping, is_neox: bool = False):
    """RoPE on ``q_pe [T,H,64]`` / ``k_pe [T,64]`` in place + insert ``[kv_c | k_pe]`` into the bf16 MLA cache."""
    if _cuda(q_pe):
        torch.ops.b200.mla_rope_and_cache(q_pe, k_pe, kv_c, mla_cache, cos_sin_cache, positions, slot_mapping, is_neox)
        return
    T, H, _ = q_pe.shape
    qo, ko = ref.rotary_embedding(positions, q_pe.reshape(T, H * 64), k_pe.reshape(T, 64), 64, cos_sin_cache, is_neox)
    q_pe.copy_(qo.reshape(T, H, 64))
    k_pe.copy_(ko.reshape(k_pe.shape))
    ops.concat_and_cache_mla(kv_c, k_pe.reshape(T, 64), mla_cache, slot_mapping)


def concat_mla_q(ql_nope: torch.Tensor, q_pe: torch.Tensor) -> torch.Tensor:
    if _cuda(ql_nope):
        out = torch.empty(*ql_nope.shape[:2], 576, dtype=ql_nope.dtype, device=ql_nope.device)
        torch.ops.b200.concat_mla_q(out, ql_nope, q_pe)
        return out
    return torch.cat([ql_nope, q_pe], dim=-1)


def permute_cols(a: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    if _cuda(a):
        out = torch.empty(a.shape[0], perm.numel(), dtype=a.dtype, device=a.device)
        torch.ops.b200.permute_cols(out, a, perm.int())
        return out
    return a[:, perm.long()]


def gather_mla_cache(mla_cache, block_table, cu_seq_lens, total: int, dtype=torch.bfloat16, seq_starts=None):
    """Paged latent cache -> contiguous ``[total, 576]`` (656-byte fp8 records are up-converted)."""
    if _cuda(mla_cache):
        dst = torch.empty(total, 576, dtype=dtype, device=mla_cache.device)
        torch.ops.b200.gather_mla_cache(dst, mla_cache, block_table, cu_seq_lens, seq_starts)
        return dst
    outs = []
    cu = cu_seq_lens.tolist()
    for b in range(len(cu) - 1):
        start = int(seq_starts[b]) if seq_starts is not None else 0
        rows = ref.gather_mla_cache(mla_cache, block_table[b], start + cu[b + 1] - cu[b])[start:]
        outs.append(rows)
    return torch.cat(outs, 0).to(dtype)


def gather_indexer_k(idx_cache, block_table, cu_seq_lens, total: int, block_size: int):
    """Paged indexer K -> ``(k fp8-as-uint8 [total,128], scale f32 [total])``."""
    if _cuda(idx_cache):
        k = torch.empty(total, 128, dtype=torch.uint8, device=idx_cache.device)
        s = torch.empty(total, dtype=torch.float32, device=idx_cache.device)
        torch.ops.b200.gather_indexer_k(k, s, idx_cache, block_table, cu_seq_lens, block_size)
        return k, s
    ks, ss = [], []
    cu = cu_seq_lens.tolist()
    flat = idx_cache.reshape(idx_cache.shape[0], -1)
    for b in range(len(cu) - 1):
        L = cu[b + 1] - cu[b]
        nblk = (L + block_size - 1) // block_size
        blk = flat[block_table[b, :nblk].long()]
        ks.append(blk[:, : block_size * 128].reshape(nblk * block_size, 128)[:L])
        ss.append(blk[:, block_size * 128:].contiguous().view(torch.float32).reshape(nblk * block_size)[:L])
    return torch.cat(ks, 0), torch.cat(ss, 0)


def selective_scan_fwd(u, delta, A, B, C, D=None, z=None, delta_bias=None, delta_softplus: bool = False,
                       ssm_states: Optional[torch.Tensor] = None, query_start_loc=None, cache_indices=None,
                       has_initial_state=None, pad_slot_id: int = -1):
    """Mamba-1 scan.  Dense: ``u [b,d,L]``, ``B/C [b,g,n,L]``; varlen: ``u [d,T]``, ``B/C [g,n,T]`` with
    ``query_start_loc``.  ``ssm_states [slots,d,n]`` fp32 is read (where ``has_initial_state``) and updated."""
    varlen = query_start_loc is not None
    batch = (query_start_loc.numel() - 1) if varlen else u.shape[0]
    d, n = A.shape
    if ssm_states is None:
        ssm_states = torch.zeros(batch, d, n, dtype=torch.float32, device=u.device)
    if _cuda(u):
        out = torch.empty_like(u)
        torch.ops.b200.selective_scan(out, u.contiguous(), delta.contiguous(), A.float().contiguous(), B.contiguous(),
                                      C.contiguous(), None if D is None else D.float(), None if z is None else z.contiguous(),
                                      None if delta_bias is None else delta_bias.float(), delta_softplus, ssm_states,
                                      query_start_loc, cache_indices,
                                      None if has_initial_state is None else has_initial_state.to(torch.uint8), pad_slot_id)
        return out, ssm_states
    out = torch.empty_like(u)
    qsl = query_start_loc.tolist() if varlen else None
    for b in range(batch):
        slot = int(cache_indices[b]) if cache_indices is not None else b
        if slot == pad_slot_id:
            continue
        if varlen:
            sl = slice(qsl[b], qsl[b + 1])
            ub, db = u[None, :, sl], delta[None, :, sl]
            Bb, Cb = B[None, :, :, sl], C[None, :, :, sl]
            zb = None if z is None else z[None, :, sl]
        else:
            ub, db, Bb, Cb = u[b:b + 1], delta[b:b + 1], B[b:b + 1], C[b:b + 1]
            zb = None if z is None else z[b:b + 1]
        g = Bb.shape[1]
        Bx = Bb.repeat_interleave(d // g, dim=1)      # [1, d, n, L] per-channel view of the group's B / C
        Cx = Cb.repeat_interleave(d // g, dim=1)
        init = ssm_states[slot:slot + 1] if (has_initial_state is not None and bool(has_initial_state[b])) else None
        y, h = _scan_per_channel(ub, db, A, Bx, Cx, D, zb, delta_bias, delta_softplus, init)
        if varlen:
            out[:, sl] = y[0]
        else:
            out[b] = y[0]
        ssm_states[slot] = h[0]
    return out, ssm_states


def _scan_per_channel(u, delta, A, B, C, D, z, delta_bias, softplus, state):
    """fp32 oracle with per-channel ``B/C [b, d, n, L]``."""
    import torch.nn.functional as F

    b, d, L = u.shape
    dl = delta.float()
    if delta_bias is not None:
        dl = dl + delta_bias.float()[None, :, None]
    if softplus:
        dl = F.softplus(dl)
    h = torch.zeros(b, d, A.shape[1]) if state is None else state.float().clone()
    ys = []
    for t in range(L):
        h = torch.exp(dl[:, :, t, None] * A.float()[None]) * h + dl[:, :, t, None] * B.float()[..., t] * u.float()[:, :, t, None]
        ys.append((h * C.float()[..., t]).sum(-1))
    y = torch.stack(ys, -1)
    if D is not None:
        y = y + u.float() * D.float()[None, :, None]
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(u.dtype), h
