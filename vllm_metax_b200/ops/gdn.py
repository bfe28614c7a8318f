"""Gated delta rule linear attention (``csrc/gdn.cu``) with its fp32 PyTorch statement.

    S <- exp(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T (scale q_t)

``q, k [T, Hq, 128]``, ``v [T, Hv, 128]`` (``Hv`` a multiple of ``Hq``), ``g, beta [T, Hv]``; sequences are given by
``query_start_loc``; ``state [slots, Hv, 128, 128]`` (fp32) is read where ``has_initial_state`` says so and always
written back at ``state_indices`` (negative index: no state is kept).
Parity: ``ChunkGatedDeltaRule`` / the fused recurrent decode step of the GDN blocks
(vllm_metax/registry/custom_ops/layers/mamba/qwen_gdn_linear_attn.py:16-88).
"""
from __future__ import annotations

from typing import Optional

import torch


def gated_delta_rule_ref(q, k, v, g, beta, query_start_loc, state=None, state_indices=None, has_initial_state=None,
                         scale: Optional[float] = None, l2norm: bool = True):
    T, Hq, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    scale = Dk ** -0.5 if scale is None else scale
    qf, kf, vf = q.float(), k.float(), v.float()
    if l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    rep = Hv // Hq
    qf, kf = qf.repeat_interleave(rep, 1) * scale, kf.repeat_interleave(rep, 1)
    out = torch.zeros(T, Hv, Dv)
    qsl = query_start_loc.tolist()
    for b in range(len(qsl) - 1):
        slot = int(state_indices[b]) if state_indices is not None else -1
        use = slot >= 0 and state is not None and (has_initial_state is None or bool(has_initial_state[b]))
        S = state[slot].float().clone() if use else torch.zeros(Hv, Dk, Dv)
        for t in range(qsl[b], qsl[b + 1]):
            S = S * torch.exp(g[t].float())[:, None, None]
            u = beta[t].float()[:, None] * (vf[t] - torch.einsum("hkv,hk->hv", S, kf[t]))
            S = S + torch.einsum("hk,hv->hkv", kf[t], u)
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        if slot >= 0 and state is not None:
            state[slot] = S.to(state.dtype)
    return out.to(q.dtype)


def gated_delta_rule_chunked(q, k, v, g, beta, query_start_loc, state=None, state_indices=None,
                             has_initial_state=None, scale: Optional[float] = None, l2norm: bool = True,
                             chunk: int = 64):
    """The same recurrence in chunked (matrix) form: inside a chunk of ``C`` tokens the updates are solved together,
    only the chunk-to-chunk state hand-over is sequential, and everything is matrix products over
    ``[heads, chunks, C, 128]`` tensors - the form prefill wants (long prompts: ``T / C`` sequential steps of a few
    batched products instead of ``T`` dependent steps).  Any device; fp32.

    With ``G_i`` the cumulative log-decay inside the chunk, ``D_ij = exp(G_i - G_j)`` (j <= i), ``S_0`` the state the
    chunk starts from:

        A   = strict-lower(diag(beta) (K K^T * D))
        T   = (I + A)^-1                                   (unit lower triangular solve, all chunks at once)
        W_v = T diag(beta) V,   W_k = T diag(beta exp(G)) K
        U   = W_v - W_k S_0                                 (the delta-rule updates of the chunk)
        O   = exp(G) * (Q S_0) + lower(Q K^T * D) U
        S_C = exp(G_C) S_0 + (K * exp(G_C - G))^T U

    Parity: the chunked kernels behind ``ChunkGatedDeltaRule``
    (vllm_metax/registry/custom_ops/layers/mamba/qwen_gdn_linear_attn.py:16-88 dispatches to them for prefill)."""
    T, Hq, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    dev = q.device
    scale = Dk ** -0.5 if scale is None else scale
    qf, kf, vf = q.float(), k.float(), v.float()
    if l2norm:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    rep = Hv // Hq
    qf, kf = qf.repeat_interleave(rep, 1) * scale, kf.repeat_interleave(rep, 1)
    gf, bf = g.float(), beta.float()
    out = torch.zeros(T, Hv, Dv, dtype=torch.float32, device=dev)
    qsl = query_start_loc.tolist()
    C = chunk
    low = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev), -1)
    eye = torch.eye(C, dtype=torch.float32, device=dev)
    for b in range(len(qsl) - 1):
        t0, t1 = qsl[b], qsl[b + 1]
        L = t1 - t0
        slot = int(state_indices[b]) if state_indices is not None else -1
        use = slot >= 0 and state is not None and (has_initial_state is None or bool(has_initial_state[b]))
        S = state[slot].float().clone() if use else torch.zeros(Hv, Dk, Dv, dtype=torch.float32, device=dev)
        if L == 0:
            continue
        N = (L + C - 1) // C
        pad = N * C - L

        def chunks(x, width):                 # [L, H, width] -> [H, N, C, width]; padding rows change nothing
            if pad:
                x = torch.cat([x, torch.zeros(pad, *x.shape[1:], dtype=x.dtype, device=dev)])
            return x.view(N, C, Hv, width).permute(2, 0, 1, 3)

        Q, K, V = chunks(qf[t0:t1], Dk), chunks(kf[t0:t1], Dk), chunks(vf[t0:t1], Dv)
        G = chunks(gf[t0:t1, :, None], 1)[..., 0].cumsum(-1)               # [H, N, C]
        B = chunks(bf[t0:t1, :, None], 1)[..., 0]
        diff = G[..., :, None] - G[..., None, :]                            # G_i - G_j
        D = torch.exp(diff.masked_fill(~low, float("-inf")))                # 0 above the diagonal
        KK = K @ K.transpose(-1, -2)
        A = (B[..., :, None] * KK * D).masked_fill(~strict, 0.0)
        Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
        Wv = Tm @ (B[..., None] * V)                                        # [H, N, C, Dv]
        Wk = Tm @ ((B * torch.exp(G))[..., None] * K)                       # [H, N, C, Dk]
        M = (Q @ K.transpose(-1, -2)) * D                                   # lower(Q K^T * D), diagonal included
        eG = torch.exp(G)
        tail = torch.exp(G[..., -1:] - G)                                   # exp(G_C - G_j)
        o_chunks = []
        for n in range(N):                                                  # the only sequential part
            U = Wv[:, n] - Wk[:, n] @ S                                     # [H, C, Dv]
            o_chunks.append(eG[:, n, :, None] * (Q[:, n] @ S) + M[:, n] @ U)
            S = eG[:, n, -1, None, None] * S + (K[:, n] * tail[:, n, :, None]).transpose(-1, -2) @ U
        O = torch.stack(o_chunks, 1)                                        # [H, N, C, Dv]
        out[t0:t1] = O.permute(1, 2, 0, 3).reshape(N * C, Hv, Dv)[:L]
        if slot >= 0 and state is not None:
            state[slot] = S.to(state.dtype)
    return out.to(q.dtype)


def gated_delta_rule(q, k, v, g, beta, query_start_loc, state=None, state_indices=None, has_initial_state=None,
                     scale: Optional[float] = None, l2norm: bool = True):
    """Output ``[T, Hv, 128]``; ``state`` is updated in place.  ``B200_GDN_CHUNKED=1`` sends batches that contain a
    prompt chunk of ``B200_GDN_CHUNKED_MIN_TOKENS`` tokens or more through the chunked form instead of the recurrent
    kernel."""
    from .. import envs

    if envs.B200_GDN_CHUNKED and q.shape[0] >= envs.B200_GDN_CHUNKED_MIN_TOKENS:
        lens = (query_start_loc[1:] - query_start_loc[:-1])
        if int(lens.max()) >= envs.B200_GDN_CHUNKED_MIN_TOKENS:
            return gated_delta_rule_chunked(q, k, v, g, beta, query_start_loc, state, state_indices, has_initial_state,
                                            scale, l2norm)
    if not q.is_cuda:
        return gated_delta_rule_ref(q, k, v, g, beta, query_start_loc, state, state_indices, has_initial_state, scale, l2norm)
    from .. import _custom_ops as ops

    ops.load_native()
    Hv = v.shape[1]
    if state is None:
        state = torch.zeros(1, Hv, 128, 128, dtype=torch.float32, device=q.device)
        state_indices = None
    out = torch.empty_like(v)
    ops._launches += 1
    torch.ops.b200.gdn_recurrent(
        out, state, q, k, v, g.float().contiguous(), beta.float().contiguous(), query_start_loc.int().contiguous(),
        None if state_indices is None else state_indices.int().contiguous(),
        None if has_initial_state is None else has_initial_state.int().contiguous(),
        q.shape[-1] ** -0.5 if scale is None else scale, l2norm)
    return out


# ------------------------------------------------------------------------------------------ short causal convolution
def causal_conv1d_ref(x, w, bias=None, state=None, query_start_loc=None, state_indices=None, has_initial_state=None,
                      silu: bool = True):
    """fp32 statement of ``csrc/causal_conv1d.cu``: ``x [T, C]``, ``w [C, K]``, ``state [slots, K-1, C]`` (oldest first,
    updated in place)."""
    T, C = x.shape
    K = w.shape[1]
    out = torch.empty(T, C, dtype=torch.float32)
    qsl = query_start_loc.tolist()
    wf = w.float()
    for b in range(len(qsl) - 1):
        s, e = qsl[b], qsl[b + 1]
        if e <= s:
            continue
        slot = int(state_indices[b]) if state_indices is not None else -1
        use = slot >= 0 and state is not None and (has_initial_state is None or bool(has_initial_state[b]))
        carry = state[slot].float() if use else torch.zeros(K - 1, C)
        ext = torch.cat([carry, x[s:e].float()], 0)                     # [K-1 + n, C]
        win = ext.unfold(0, K, 1)                                       # [n, C, K]
        y = (win * wf[None]).sum(-1)
        if bias is not None:
            y = y + bias.float()
        out[s:e] = torch.nn.functional.silu(y) if silu else y
        if slot >= 0 and state is not None:
            state[slot] = ext[-(K - 1):].to(state.dtype)
    return out.to(x.dtype)


def causal_conv1d(x, w, bias=None, state=None, query_start_loc=None, state_indices=None, has_initial_state=None,
                  silu: bool = True):
    """Depthwise causal convolution (+ SiLU) over a ragged batch; the last ``K-1`` inputs of every sequence are carried
    in ``state`` between steps.  Parity: the ``causal_conv1d_fn`` / ``causal_conv1d_update`` pair the reference's GDN
    layer calls (vllm_metax/registry/custom_ops/layers/mamba/qwen_gdn_linear_attn.py:8-10)."""
    if not x.is_cuda:
        return causal_conv1d_ref(x, w, bias, state, query_start_loc, state_indices, has_initial_state, silu)
    from .. import _custom_ops as ops

    ops.load_native()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    ops._launches += 2 if state is not None else 1
    torch.ops.b200.causal_conv1d(out, x, w.contiguous(), bias, state, query_start_loc.int().contiguous(),
                                 None if state_indices is None else state_indices.int().contiguous(),
                                 None if has_initial_state is None else has_initial_state.int().contiguous(), silu)
    return out
