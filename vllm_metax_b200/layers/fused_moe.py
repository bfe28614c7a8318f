"""Mixture-of-experts layer: routing -> (EP dispatch) -> grouped expert GEMMs -> combine.

Data flow on one rank (bf16):

    router logits  = x @ W_gate^T                      tcgen05 GEMM
    (w, ids)       = fused score + top-k               one warp per token
    align          = expert-sort of the (token, k) pairs, padded to 128 rows per expert
    A_perm         = gather(x)                         expert-contiguous rows
    H              = grouped GEMM(A_perm, w13)         SiLU-gate fused in the epilogue
    Y              = grouped GEMM(H, w2)
    out            = sum_k w_k * Y[pos(t, k)] (+ shared expert)

Weights: ``w13 [E_local, 2I, H]`` with gate/up rows interleaved (row 2j = gate_j, 2j+1 = up_j),
``w2 [E_local, H, I]``.

Expert parallelism: experts are sharded over the EP group (``E_local = E / ep``).  Tokens are
replicated across the TP/EP ranks in this engine (SPMD, attention is tensor-parallel), so
"dispatch" is a local filter - every rank gathers the pairs routed to ITS experts
(``expert_map``) - and "combine" is a sum over ranks of the partial outputs, which is exactly the
row-parallel reduction and is therefore fused with the residual add + RMSNorm in
``parallel/fused_collectives.py`` (or falls back to an NCCL all-reduce).  Data-parallel
attention (tokens differ per rank) goes through ``parallel/all2all.py``.

Parity: vllm_metax/model_executor/layers/fused_moe/fused_moe.py:1960-2436 (fused_experts),
experts/triton_moe.py:221-620, all2all_utils.py:34-126.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _custom_ops as ops
from .. import envs
from ..ops import reference as ref
from ..parallel import state as ps
from .linear import ReplicatedLinear

BLOCK_M = 128


def fused_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor, num_local_experts: int, expert_map: Optional[torch.Tensor] = None,
                  shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expert MLPs for the pairs routed to this rank's experts; returns ``[T, H]`` (partial sum
    when ``expert_map`` drops pairs owned by other ranks)."""
    T, H = x.shape
    topk = topk_ids.shape[1]
    sorted_ids, block_expert, total, inv = ops.moe_align_block_size(topk_ids, BLOCK_M, num_local_experts,
                                                                    expert_map, want_inverse=True)
    a = ops.moe_gather(x, sorted_ids, total, topk)
    h = ops.gemm_grouped(a, w13, block_expert, total, epi=1)
    y = ops.gemm_grouped(h, w2, block_expert, total, epi=0)
    return ops.moe_combine(y, topk_weights, inv, T, shared_out)


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 dtype=torch.bfloat16, renormalize: bool = True, scoring_func: str = "softmax",
                 use_grouped_topk: bool = False, num_expert_group: int = 1, topk_group: int = 1,
                 routed_scaling_factor: float = 1.0, e_score_correction_bias: bool = False,
                 reduce_results: bool = True, quant_method=None, prefix: str = ""):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.renormalize, self.scoring_func = renormalize, scoring_func
        self.use_grouped_topk, self.num_expert_group, self.topk_group = use_grouped_topk, num_expert_group, topk_group
        self.routed_scaling_factor = routed_scaling_factor
        self.reduce_results = reduce_results
        self.prefix = prefix
        # experts are sharded over the TP group's ranks (TP == EP in this engine)
        self.ep = ps.tp_size()
        self.ep_rank = ps.tp_rank()
        assert num_experts % self.ep == 0, "number of experts must divide over the EP ranks"
        self.num_local = num_experts // self.ep
        self.quant_method = quant_method
        if quant_method is not None:
            quant_method.create_weights(self, self.num_local, hidden_size, intermediate_size, dtype)
        else:
            self.w13_weight = nn.Parameter(torch.empty(self.num_local, 2 * intermediate_size, hidden_size, dtype=dtype),
                                           requires_grad=False)
            self.w2_weight = nn.Parameter(torch.empty(self.num_local, hidden_size, intermediate_size, dtype=dtype),
                                          requires_grad=False)
        self.e_score_correction_bias = (nn.Parameter(torch.zeros(num_experts, dtype=torch.float32), requires_grad=False)
                                        if e_score_correction_bias else None)
        if self.ep > 1:
            emap = torch.full((num_experts,), -1, dtype=torch.int32)
            lo = self.ep_rank * self.num_local
            emap[lo: lo + self.num_local] = torch.arange(self.num_local, dtype=torch.int32)
            self.register_buffer("expert_map", emap, persistent=False)
        else:
            self.expert_map = None

    # ---- weights ----------------------------------------------------------------
    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, expert_id: Optional[int] = None,
                      shard: Optional[str] = None) -> None:
        """``shard`` in {w1 (gate), w3 (up), w2 (down)}; ``expert_id`` is global.  Without an expert id the tensor is a
        per-layer one (the routing bias) and is copied as is."""
        if expert_id is None:
            param.data.copy_(loaded.reshape(param.shape))
            return
        lo = self.ep_rank * self.num_local
        if not (lo <= expert_id < lo + self.num_local):
            return
        e = expert_id - lo
        if self.quant_method is not None and hasattr(self.quant_method, "load_expert_weight"):
            self.quant_method.load_expert_weight(self, param, loaded, e, shard)
            return
        if shard == "w1":
            param.data[e, 0::2].copy_(loaded)
        elif shard == "w3":
            param.data[e, 1::2].copy_(loaded)
        else:
            param.data[e].copy_(loaded)

    def load_expert_tensor(self, expert_id: int, shard: str, suffix: str, loaded: torch.Tensor) -> bool:
        """Checkpoint tensors that have no one-to-one parameter (packed weight-only formats): the quant
        method converts them.  Returns False when the tensor is not consumed."""
        qm = self.quant_method
        if qm is None or not hasattr(qm, "load_expert_tensor"):
            return False
        lo = self.ep_rank * self.num_local
        if lo <= expert_id < lo + self.num_local:
            qm.load_expert_tensor(self, expert_id - lo, shard, suffix, loaded)
        return True

    # ---- forward ------------------------------------------------------------------
    def route(self, router_logits: torch.Tensor):
        bias = self.e_score_correction_bias
        if self.use_grouped_topk:
            return ops.grouped_topk(router_logits, self.top_k, self.renormalize, self.num_expert_group,
                                    self.topk_group, self.scoring_func, bias, self.routed_scaling_factor)
        return ops.topk_gating(router_logits, self.top_k, self.renormalize, self.scoring_func, bias,
                               self.routed_scaling_factor)

    def _forward_a2a(self, x: torch.Tensor, router_logits: torch.Tensor,
                     shared_out: Optional[torch.Tensor]) -> torch.Tensor:
        """Sequence-parallel MoE over the NVLink dispatch / combine kernels: every rank routes its own 1/ep of the
        tokens, rows travel once to the ranks that own their experts, partial sums come back, and the finished rows
        are all-gathered - instead of every rank running its experts on all tokens and all-reducing ``[T, H]``
        (the reference's sequence-parallel MoE region, models/deepseek_v2.py:1286-1316, with its all2all managers)."""
        from ..parallel.all2all import NvlinkAll2AllManager, run_experts_a2a

        g = ps.get_tp_group()
        T, H = x.shape
        per = (T + self.ep - 1) // self.ep
        sizes = [max(0, min(per, T - r * per)) for r in range(self.ep)]
        lo, n = self.ep_rank * per, sizes[self.ep_rank]
        qm = self.quant_method
        wire_fp8 = bool(getattr(qm, "a2a_wire_fp8", False))
        mgr = getattr(self, "_a2a", None)
        if mgr is None or mgr.max_tokens < per:
            if mgr is not None:
                mgr.close()
            cap = max(per, 64)
            mgr = NvlinkAll2AllManager(g, cap, H, self.top_k, self.num_experts, x.dtype, x.device, quant_fp8=wire_fp8)
            self._a2a = mgr
        if n > 0:
            w, ids = self.route(router_logits[lo: lo + n])
        else:           # fewer tokens than ranks: this rank only serves its experts
            w = torch.empty(0, self.top_k, dtype=torch.float32, device=x.device)
            ids = torch.empty(0, self.top_k, dtype=torch.int32, device=x.device)

        def experts(a, a_scale, block_expert, total):
            if qm is not None:
                return qm.apply_sorted(self, a, a_scale, block_expert, total)
            h = ops.gemm_grouped(a, self.w13_weight, block_expert, total, epi=1)
            return ops.gemm_grouped(h, self.w2_weight, block_expert, total)

        mine = run_experts_a2a(mgr, x[lo: lo + n].contiguous(), w, ids, experts)
        y = g.all_gatherv(mine, sizes)
        if shared_out is not None:       # shared experts are tensor-parallel: their partial sums still need the reduction
            y = y + (ps.tensor_model_parallel_all_reduce(shared_out) if self.reduce_results else shared_out)
        return y

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor,
                shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if (self.ep > 1 and (self.quant_method is None or hasattr(self.quant_method, "apply_sorted"))
                and self.reduce_results and x.is_cuda and envs.B200_MOE_A2A and x.shape[1] % 128 == 0):
            return self._forward_a2a(x, router_logits, shared_out)
        w, ids = self.route(router_logits)
        if self.quant_method is not None:
            y = self.quant_method.apply(self, x, w, ids, shared_out)
        else:
            y = fused_experts(x, self.w13_weight, self.w2_weight, w, ids, self.num_local, self.expert_map, shared_out)
        if self.reduce_results and self.ep > 1:
            y = ps.tensor_model_parallel_all_reduce(y)
        return y


def reference_moe(x, w13, w2, topk_weights, topk_ids):
    """fp32 oracle on the interleaved-w13 layout."""
    gate, up = w13[:, 0::2], w13[:, 1::2]
    return ref.fused_experts(x, torch.cat([gate, up], dim=1), w2, topk_weights, topk_ids)
