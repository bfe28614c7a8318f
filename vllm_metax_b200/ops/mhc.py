"""Manifold hyper-connection (mHC) ops of DeepSeek-V4: CUDA kernels (``csrc/mhc.cu``) for CUDA tensors, the fp32
PyTorch statement of the same math otherwise (also the test oracle).

The residual is ``M`` parallel streams ``[T, M, H]``.  ``mhc_pre`` derives, per token, the read weights
(``pre``), write weights (``post``) and the doubly-stochastic stream-mixing matrix (``comb``, Sinkhorn) from
the RMS-normalised streams, and returns the sub-layer input ``x = sum_i pre_i * stream_i``.  ``mhc_post`` writes
a sub-layer output back: ``stream'_n = y * post_n + sum_m comb[m, n] * stream_m``.
Parity: vllm_metax/models/deepseek_v4/ops/mhc/torch.py:10-299, tilelang_kernels.py:45-356.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _custom_ops as ops


def sinkhorn(x: torch.Tensor, iters: int, eps: float) -> torch.Tensor:
    x = x.softmax(-1) + eps
    x = x / (x.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        x = x / (x.sum(-1, keepdim=True) + eps)
        x = x / (x.sum(-2, keepdim=True) + eps)
    return x


def _mixes(residual, fn, rms_eps):
    T, M, H = residual.shape
    r = residual.reshape(T, M * H).float()
    inv = torch.rsqrt(r.square().mean(-1, keepdim=True) + rms_eps)
    return (r @ fn.float().t()) * inv


def mhc_pre_ref(residual, fn, scale, base, rms_eps, pre_eps, sinkhorn_eps, post_mult, iters):
    T, M, H = residual.shape
    mixes = _mixes(residual, fn, rms_eps)
    sc = torch.cat([scale[0].expand(M), scale[1].expand(M), scale[2].expand(M * M)]).float()
    mixes = mixes * sc + base.float()
    pre = torch.sigmoid(mixes[:, :M]) + pre_eps
    post = torch.sigmoid(mixes[:, M:2 * M]) * post_mult
    comb = sinkhorn(mixes[:, 2 * M:].reshape(T, M, M), iters, sinkhorn_eps)
    x = (residual.float() * pre[:, :, None]).sum(1).to(residual.dtype)
    return post, comb, x


def mhc_post_ref(y, residual, post, comb):
    out = y.float()[:, None, :] * post[:, :, None] + torch.einsum("tmn,tmh->tnh", comb, residual.float())
    return out.to(residual.dtype)


def mhc_head_ref(residual, fn, scale, base, rms_eps, pre_eps):
    mixes = _mixes(residual, fn, rms_eps) * scale.float()[0] + base.float()
    pre = torch.sigmoid(mixes) + pre_eps
    return (residual.float() * pre[:, :, None]).sum(1).to(residual.dtype)


def mhc_pre(residual, fn, scale, base, rms_eps: float, pre_eps: float, sinkhorn_eps: float, post_mult: float,
            iters: int):
    """-> ``(post [T,M] f32, comb [T,M,M] f32, x [T,H])``."""
    if ops._use_cuda(residual):
        T, M, H = residual.shape
        dev = residual.device
        post = torch.empty(T, M, dtype=torch.float32, device=dev)
        comb = torch.empty(T, M, M, dtype=torch.float32, device=dev)
        x = torch.empty(T, H, dtype=residual.dtype, device=dev)
        torch.ops.b200.mhc_pre(x, post, comb, residual, None, None, None, None, fn, scale, base, rms_eps, pre_eps,
                               sinkhorn_eps, post_mult, iters, False)
        return post, comb, x
    return mhc_pre_ref(residual, fn, scale, base, rms_eps, pre_eps, sinkhorn_eps, post_mult, iters)


def mhc_post(y, residual, post, comb):
    if ops._use_cuda(residual):
        out = torch.empty_like(residual)
        torch.ops.b200.mhc_post(out, y.contiguous(), residual, post, comb)
        return out
    return mhc_post_ref(y, residual, post, comb)


def mhc_fused_post_pre(y, residual, post, comb, fn, scale, base, rms_eps, pre_eps, sinkhorn_eps, post_mult, iters,
                       out: Optional[torch.Tensor] = None):
    """``post`` of the finished sub-layer and ``pre`` of the next in one pass.
    -> ``(new_residual, post', comb', x)``."""
    if ops._use_cuda(residual):
        T, M, H = residual.shape
        dev = residual.device
        new_res = torch.empty_like(residual) if out is None else out
        post2 = torch.empty(T, M, dtype=torch.float32, device=dev)
        comb2 = torch.empty(T, M, M, dtype=torch.float32, device=dev)
        x = torch.empty(T, H, dtype=residual.dtype, device=dev)
        torch.ops.b200.mhc_pre(x, post2, comb2, residual, new_res, y.contiguous(), post, comb, fn, scale, base, rms_eps,
                               pre_eps, sinkhorn_eps, post_mult, iters, False)
        return new_res, post2, comb2, x
    new_res = mhc_post_ref(y, residual, post, comb)
    return (new_res,) + tuple(mhc_pre_ref(new_res, fn, scale, base, rms_eps, pre_eps, sinkhorn_eps, post_mult, iters))


def mhc_head(residual, fn, scale, base, rms_eps: float, pre_eps: float):
    """Final mix before the output norm: ``M`` read weights only."""
    if ops._use_cuda(residual):
        T, M, H = residual.shape
        x = torch.empty(T, H, dtype=residual.dtype, device=residual.device)
        torch.ops.b200.mhc_pre(x, None, None, residual, None, None, None, None, fn, scale, base, rms_eps, pre_eps, 0.0,
                               1.0, 1, True)
        return x
    return mhc_head_ref(residual, fn, scale, base, rms_eps, pre_eps)


def expand_to_streams(hidden: torch.Tensor, m: int) -> torch.Tensor:
    return hidden.unsqueeze(1).expand(hidden.shape[0], m, hidden.shape[1]).contiguous()
