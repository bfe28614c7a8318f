"""Fused compute + collective layers over NVLink peer memory.

``FusedRowParallelNorm`` is the tensor-parallel row-parallel linear (o_proj / down_proj) fused
with everything that follows it: GEMM -> reduce-scatter into the owning rank -> residual add
-> RMSNorm -> all-gather of the normalised rows, as ONE kernel per rank
(``csrc/comm_gemm_ar_norm.cu``).  It replaces GEMM + NCCL all-reduce + fused_add_rms_norm
(the reference's path C1 -> K12, and its quick-reduce / minimax_reduce_rms special cases).

The residual stream is kept sharded by token rows between calls: rank r owns rows
``[r * rows_per_rank, (r + 1) * rows_per_rank)`` of the step's ``T`` tokens.

On CPU tensors (Gloo ranks) the same contract is met with plain collectives, which is how the
host-side logic is tested without GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _custom_ops as ops
from .. import envs
from ..ops import reference as ref
from .state import Group
from .symm_mem import SymmWorkspace


def rows_per_rank(T: int, tp: int) -> int:
    return (T + tp - 1) // tp


class FusedRowParallelNorm:
    """Workspace + launcher shared by every fused row-parallel layer of a model."""

    def __init__(self, group: Group, device: torch.device, max_tokens: int, hidden: int, dtype: torch.dtype):
        self.group, self.device, self.hidden, self.dtype = group, device, hidden, dtype
        self.tp, self.rank = group.world_size, group.rank_in_group
        self.max_tokens = max_tokens
        self.rows_cap = (rows_per_rank(max_tokens, self.tp) + 7) // 8 * 8
        self.rb_cap = (max_tokens + 127) // 128 + 1
        self.cuda = device.type == "cuda"
        if not self.cuda:
            return
        esz = torch.empty((), dtype=dtype).element_size()
        n_recv = self.tp * self.rows_cap * hidden * esz
        n_out = max_tokens * hidden * esz
        n_cnt = 2 * self.rb_cap * 4
        n_flag = 64
        self.ws = SymmWorkspace(group, n_recv + n_out + n_cnt + n_flag + 8 * SymmWorkspace.ALIGN, device)
        r_recv = self.ws.region("recv", n_recv)
        r_cnt = self.ws.region("counters", n_cnt)
        r_flag = self.ws.region("flags", n_flag)
        r_out = self.ws.region("out", n_out)
        self.out = self.ws.local(r_out, dtype, (max_tokens, hidden))
        self.ptrs = torch.tensor([self.ws.peer_ptrs(r_recv), self.ws.peer_ptrs(r_cnt), self.ws.peer_ptrs(r_flag),
                                  self.ws.peer_ptrs(r_out)], dtype=torch.int64)
        self.local_sync = torch.zeros(4, dtype=torch.int32, device=device)
        self.wait_cycles = int(envs.B200_PEER_WAIT_ITERS) * 200  # iteration budget expressed in SM cycles
        torch.cuda.synchronize(device)
        group.barrier()

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, residual_shard: torch.Tensor,
                 norm_weight: torch.Tensor, eps: float, add_residual: bool = True) -> torch.Tensor:
        """``x [T, K_local]``, ``weight [H, K_local]``; ``residual_shard [rows_per_rank(T), H]`` is updated in
        place (overwritten when ``add_residual`` is False).  Returns the normalised ``[T, H]`` (a view of the
        symmetric output buffer, valid until the next call)."""
        T = x.shape[0]
        rpr = rows_per_rank(T, self.tp)
        if self.cuda:
            assert T <= self.max_tokens
            ops._launches += 1
            torch.ops.b200.gemm_ar_norm(x, weight, residual_shard, norm_weight, eps, self.ptrs, self.tp, self.rank,
                                        rpr, self.rows_cap, self.rb_cap, self.local_sync, add_residual,
                                        self.wait_cycles)
            return self.out[:T]
        # CPU ranks: same contract through plain collectives
        part = ref.gemm(x, weight, out_dtype=torch.float32)
        part = part.to(x.dtype).float()              # partials travel in the activation dtype
        pad = rpr * self.tp - T
        if pad:
            part = torch.cat([part, part.new_zeros(pad, part.shape[1])])
        mine = self.group.reduce_scatter(part, 0)
        my_rows = max(0, min(rpr, T - self.rank * rpr))
        if add_residual:
            mine[:my_rows] += residual_shard[:my_rows].float()
        residual_shard[:my_rows] = mine[:my_rows].to(residual_shard.dtype)
        normed = ref.rms_norm(residual_shard[:rpr], norm_weight, eps)
        if normed.shape[0] < rpr:
            normed = torch.cat([normed, normed.new_zeros(rpr - normed.shape[0], normed.shape[1])])
        return self.group.all_gather(normed.contiguous(), 0)[:T]


_SHARED: dict = {}


def get_fused_row_parallel(group: Group, device: torch.device, max_tokens: int, hidden: int,
                           dtype: torch.dtype) -> FusedRowParallelNorm:
    key = (id(group), str(device), hidden, dtype)
    cur = _SHARED.get(key)
    if cur is None or cur.max_tokens < max_tokens:
        cur = FusedRowParallelNorm(group, device, max_tokens, hidden, dtype)
        _SHARED[key] = cur
    return cur
