"""DeepSeek-V4 latent-cache records (``csrc/v4_cache.cu``) and their fp32 PyTorch statement.

Record of one token (584 bytes): 448 e4m3 values in 7 blocks of 64 with one power-of-two scale each, the 64 rotated
rope dims as bf16, then 7 UE8M0 scale bytes + 1 pad.  In a cache block the ``block_size x 576`` data bytes come first,
the ``block_size x 8`` scale bytes after them.

Parity: csrc/libtorch_stable/fused_deepseek_v4_qnorm_rope_kv_insert_kernel.cu:165-480 of the reference
(``fused_deepseek_v4_qnorm_rope_kv_rope_quant_insert``) and vllm_metax/models/deepseek_v4/ops/cache_utils.py:7.
"""
from __future__ import annotations

import torch

HEAD, ROPE, NOPE, QBLOCK = 512, 64, 448, 64
DATA_BYTES, SCALE_BYTES, RECORD_BYTES = 576, 8, 584


def alloc_cache(num_blocks: int, block_size: int, device) -> torch.Tensor:
    """``uint8 [num_blocks, block_size * 584]`` (rows padded to 16 bytes)."""
    stride = (block_size * RECORD_BYTES + 15) // 16 * 16
    return torch.zeros(num_blocks, stride, dtype=torch.uint8, device=device)


def _rope_interleaved(x: torch.Tensor, cos_sin_rows: torch.Tensor) -> torch.Tensor:
    """x [..., 64] fp32, rows [..., 64] = cos[32] | sin[32]; pairs (2i, 2i+1)."""
    cos, sin = cos_sin_rows[..., :32], cos_sin_rows[..., 32:]
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)


def qnorm_rope_kv_insert_ref(q, kv, cache, slot_mapping, positions, cos_sin, eps, block_size, hq_pad=None):
    """fp32 statement; writes records into ``cache`` (CPU or GPU tensor) and returns ``q_out [T, hq_pad, 512]``."""
    T, Hq, _ = q.shape
    hq_pad = hq_pad or Hq
    rows = cos_sin[positions[:T]].float()
    qf = q.float()
    qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + eps)
    qf = torch.cat([qf[..., :NOPE], _rope_interleaved(qf[..., NOPE:], rows[:, None, :])], -1)
    q_out = torch.zeros(T, hq_pad, HEAD, dtype=q.dtype, device=q.device)
    q_out[:, :Hq] = qf.to(q.dtype)
    n = slot_mapping.numel()
    kvf = kv[:n].float()
    kvf = torch.cat([kvf[:, :NOPE], _rope_interleaved(kvf[:, NOPE:], rows[:n])], -1).to(torch.bfloat16)
    nope = kvf[:, :NOPE].float().view(n, NOPE // QBLOCK, QBLOCK)
    amax = nope.abs().amax(-1).clamp_min(1e-4)
    ex = torch.ceil(torch.log2(amax / 448.0))
    qv = (nope * torch.exp2(-ex)[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).view(n, NOPE)
    sb = (ex + 127.0).clamp(0, 255).to(torch.uint8)
    rope_bytes = kvf[:, NOPE:].contiguous().view(torch.uint8).view(n, 2 * ROPE)
    for i in range(n):
        s = int(slot_mapping[i])
        if s < 0:
            continue
        blk, pos = divmod(s, block_size)
        row = cache[blk]
        row[pos * DATA_BYTES: pos * DATA_BYTES + NOPE] = qv[i]
        row[pos * DATA_BYTES + NOPE: (pos + 1) * DATA_BYTES] = rope_bytes[i]
        so = block_size * DATA_BYTES + pos * SCALE_BYTES
        row[so: so + 7] = sb[i]
        row[so + 7] = 0
    return q_out


def gather_dequant_ref(cache, slots, block_size):
    n = slots.numel()
    out = torch.zeros(n, HEAD, dtype=torch.bfloat16, device=cache.device)
    for i in range(n):
        s = int(slots[i])
        if s < 0:
            continue
        blk, pos = divmod(s, block_size)
        row = cache[blk]
        data = row[pos * DATA_BYTES: (pos + 1) * DATA_BYTES]
        so = block_size * DATA_BYTES + pos * SCALE_BYTES
        sc = torch.exp2(row[so: so + 7].float() - 127.0)
        vals = data[:NOPE].contiguous().view(torch.float8_e4m3fn).float().view(7, QBLOCK) * sc[:, None]
        out[i, :NOPE] = vals.flatten().to(torch.bfloat16)
        out[i, NOPE:] = data[NOPE:].contiguous().view(torch.bfloat16)
    return out


def qnorm_rope_kv_insert(q, kv, cache, slot_mapping, positions, cos_sin, eps: float, block_size: int, hq_pad=None):
    """``q [T, Hq, 512]`` -> ``q_out [T, hq_pad, 512]`` (weightless RMSNorm + interleaved RoPE on the last 64 dims, pad
    heads zero); ``kv [T, 512]`` -> RoPE, block-64 UE8M0 fp8 quantisation, record insert at ``slot_mapping`` (which may
    be shorter than T: padded tokens get no record; negative slots are skipped)."""
    if not q.is_cuda:
        return qnorm_rope_kv_insert_ref(q, kv, cache, slot_mapping, positions, cos_sin, eps, block_size, hq_pad)
    from .. import _custom_ops as ops

    ops.load_native()
    q_out = torch.empty(q.shape[0], hq_pad or q.shape[1], HEAD, dtype=q.dtype, device=q.device)
    ops._launches += 1
    torch.ops.b200.v4_qnorm_rope_kv_insert(q_out, cache, q, kv, slot_mapping.long().contiguous(),
                                           positions.long().contiguous(), cos_sin, eps, block_size)
    return q_out


def gather_dequant(cache, slots, block_size: int):
    """Records at ``slots`` as ``bf16 [n, 512]`` (negative slots give zero rows)."""
    if not cache.is_cuda:
        return gather_dequant_ref(cache, slots, block_size)
    from .. import _custom_ops as ops

    ops.load_native()
    out = torch.empty(slots.numel(), HEAD, dtype=torch.bfloat16, device=cache.device)
    ops._launches += 1
    torch.ops.b200.v4_gather_dequant(out, cache, slots.long().contiguous(), block_size)
    return out


def inv_rope(o: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, n_groups: int) -> torch.Tensor:
    """Attention output ``o [T, H, 512]`` -> ``[T, n_groups, (H / n_groups) * 512]`` with the rope dims of every head
    rotated back (inverse interleaved RoPE); storage is group-major (``[G, T, d]``, returned transposed) so that
    each group's slab feeds one GEMM of the grouped output projection."""
    T, H, _ = o.shape
    hpg = H // n_groups
    if o.is_cuda:
        from .. import _custom_ops as ops

        ops.load_native()
        out = torch.empty(n_groups, T, hpg * HEAD, dtype=o.dtype, device=o.device)
        ops._launches += 1
        torch.ops.b200.v4_inv_rope(out, o, positions.long().contiguous(), cos_sin, n_groups)
        return out.transpose(0, 1)
    rows = cos_sin[positions[:T]].float()[:, None, :]
    cos, sin = rows[..., :32], rows[..., 32:]
    x = o.float()
    a, b = x[..., NOPE::2], x[..., NOPE + 1::2]
    rot = torch.stack((a * cos + b * sin, b * cos - a * sin), dim=-1).flatten(-2)
    y = torch.cat([x[..., :NOPE], rot], -1).to(o.dtype)
    return y.reshape(T, n_groups, hpg * HEAD)


def indexer_q_rope_int8_quant(positions, index_q, cos_sin, index_weights, softmax_scale: float, head_scale: float):
    """``index_q [T, H, 128]``: interleaved RoPE on the last ``cos_sin.shape[1]`` dims, int8 quantisation with one scale
    per (token, head); returns ``(q_int8 [T, H, 128], weights_out [T, H] f32)`` with
    ``weights_out = index_weights * q_scale * softmax_scale * head_scale``."""
    T, H, D = index_q.shape
    if index_q.is_cuda:
        from .. import _custom_ops as ops

        ops.load_native()
        q8 = torch.empty(T, H, D, dtype=torch.int8, device=index_q.device)
        w_out = torch.empty(T, H, dtype=torch.float32, device=index_q.device)
        ops._launches += 1
        torch.ops.b200.v4_indexer_q(q8, w_out, index_q, index_weights, positions.long().contiguous(), cos_sin,
                                    softmax_scale, head_scale)
        return q8, w_out
    rot = cos_sin.shape[1]
    rows = cos_sin[positions[:T]].float()[:, None, :]
    cos, sin = rows[..., : rot // 2], rows[..., rot // 2:]
    x = index_q.float()
    a, b = x[..., D - rot::2], x[..., D - rot + 1::2]
    r = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2).to(torch.bfloat16).float()
    x = torch.cat([x[..., : D - rot], r], -1)
    amax = x.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    v = x / scale
    q8 = torch.where(v >= 0, torch.floor(v + 0.5), torch.ceil(v - 0.5)).clamp(-127, 127).to(torch.int8)
    return q8, index_weights.float() * scale[..., 0] * softmax_scale * head_scale
