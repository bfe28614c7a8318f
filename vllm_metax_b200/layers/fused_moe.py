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

Expert parallelism: experts are sharded over the EP group (``E_local = E / ep``).

* One replica (``data_parallel_size == 1``): EP group = TP group.  Tokens are replicated across its ranks (SPMD,
  attention is tensor-parallel), so by default "dispatch" is a local filter - every rank gathers the pairs routed
  to ITS experts (``expert_map``) - and "combine" is a sum over ranks of the partial outputs, which is exactly the
  row-parallel reduction (fused with the residual add + RMSNorm in ``parallel/fused_collectives.py``, or an
  all-reduce).  With ``B200_MOE_A2A=1`` the layer instead runs sequence-parallel: every rank routes 1 / tp of the
  tokens and the rows travel once over the NVLink dispatch / combine kernels.
* Several replicas (``data_parallel_size > 1``, "DP attention + EP"): EP group = all dp x tp ranks.  Every replica
  has its own tokens; each of its TP ranks routes a slice of them, the slices are exchanged over the EP group
  (``parallel/all2all.py``: NVLink kernels, or all-gather / reduce-scatter on any backend), every rank runs its
  experts on what it received, and the results travel back.  The engines of the replicas step in lock-step
  (``engine/llm.py``) so that every rank takes part in every exchange.

``forward_reduced`` picks the path and returns the complete output; ``forward`` is the local-filter path (partial
sums when experts live on several ranks).

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
        # experts are sharded over the EP group: the TP group of a single replica, all dp x tp ranks otherwise
        self.dp = ps.get_dp_group().world_size
        self.ep_group = ps.get_ep_group() if self.dp > 1 else ps.get_tp_group()
        self.ep = self.ep_group.world_size
        self.ep_rank = self.ep_group.rank_in_group
        # load balancing: num_physical = num_experts + redundant slots; hot experts live in several slots
        self._sp_config = ps.moe_sequence_parallel()
        self.eplb = ps.eplb_enabled()
        self.num_physical = num_experts + (ps.num_redundant_experts() if self.eplb else 0)
        assert self.num_physical % self.ep == 0, "number of expert slots must divide over the EP ranks"
        self.num_local = self.num_physical // self.ep
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
            emap = torch.full((self.num_physical,), -1, dtype=torch.int32)
            lo = self.ep_rank * self.num_local
            emap[lo: lo + self.num_local] = torch.arange(self.num_local, dtype=torch.int32)
            self.register_buffer("expert_map", emap, persistent=False)
        else:
            self.expert_map = None
        if self.eplb:
            from ..parallel import eplb

            phy2log = eplb.initial_placement(num_experts, self.num_physical)
            l2p, cnt = eplb.build_maps(phy2log, num_experts, self.num_physical - num_experts + 1)
            self.register_buffer("phy2log", phy2log.to(torch.int32), persistent=False)
            self.register_buffer("log2phy", l2p, persistent=False)
            self.register_buffer("logcnt", cnt, persistent=False)
            self.register_buffer("expert_load", torch.zeros(num_experts, dtype=torch.int64), persistent=False)

    # ---- load balancing ---------------------------------------------------------
    _EPLB_BUFFERS = ("phy2log", "log2phy", "logcnt", "expert_load", "expert_map", "e_score_correction_bias")

    def _local_slots(self, expert_id: int) -> list:
        """Local slot indices that hold logical expert ``expert_id`` on this rank."""
        lo = self.ep_rank * self.num_local
        if not self.eplb:
            return [expert_id - lo] if lo <= expert_id < lo + self.num_local else []
        mine = self.phy2log[lo: lo + self.num_local].tolist()
        return [i for i, e in enumerate(mine) if e == expert_id]

    def expert_tensors(self) -> list:
        """Every per-slot tensor of this layer (first dimension = local slots): what a re-placement moves."""
        out = []
        for name, t in list(self._parameters.items()) + list(self._buffers.items()):
            if t is None or name in self._EPLB_BUFFERS:
                continue
            if t.dim() >= 1 and t.shape[0] == self.num_local:
                out.append(t.data)
        return out

    def apply_placement(self, new_phy2log: torch.Tensor) -> int:
        """Move expert weights to the slots ``new_phy2log [P]`` names and switch the routing maps; collective over the
        EP group.  Returns the number of expert rows received from other ranks."""
        from ..parallel import eplb

        old = self.phy2log.cpu().to(torch.int64)
        new = new_phy2log.to(torch.int64).cpu()
        tensors = self.expert_tensors()
        moved = 0
        if self.ep > 1:
            moved = eplb.rearrange_layer(tensors, old, new, self.ep_group.ranks, self.ep_rank,
                                         group=self.ep_group._pg(tensors[0]))
        else:
            eplb.rearrange_layer(tensors, old, new, [0], 0)
        l2p, cnt = eplb.build_maps(new, self.num_experts, self.log2phy.shape[1])
        self.phy2log.copy_(new.to(torch.int32))
        self.log2phy.copy_(l2p)
        self.logcnt.copy_(cnt)
        return moved

    def _to_physical(self, ids: torch.Tensor) -> torch.Tensor:
        """Logical expert ids ``[T, k]`` -> physical slots: the pairs of a replicated expert take its copies in turn
        (by token index), and the logical load is counted for the next re-placement."""
        flat = ids.reshape(-1).long()
        self.expert_load.scatter_add_(0, flat, torch.ones_like(flat))
        T, k = ids.shape
        turn = torch.arange(T, device=ids.device).unsqueeze(1) + torch.arange(k, device=ids.device).unsqueeze(0)
        cnt = self.logcnt[flat].view(T, k)
        rep = turn % cnt
        return self.log2phy[flat, rep.reshape(-1).long()].view(T, k).to(ids.dtype)

    # ---- weights ----------------------------------------------------------------
    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, expert_id: Optional[int] = None,
                      shard: Optional[str] = None) -> None:
        """``shard`` in {w1 (gate), w3 (up), w2 (down)}; ``expert_id`` is global.  Without an expert id the tensor is a
        per-layer one (the routing bias) and is copied as is."""
        if expert_id is None:
            param.data.copy_(loaded.reshape(param.shape))
            return
        for e in self._local_slots(expert_id):
            if self.quant_method is not None and hasattr(self.quant_method, "load_expert_weight"):
                self.quant_method.load_expert_weight(self, param, loaded, e, shard)
            elif shard == "w1":
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
        for e in self._local_slots(expert_id):
            qm.load_expert_tensor(self, e, shard, suffix, loaded)
        return True

    # ---- forward ------------------------------------------------------------------
    def route(self, router_logits: torch.Tensor):
        """``(weights, ids) [T, k]``; the ids name expert SLOTS (= experts unless load balancing replicates some)."""
        bias = self.e_score_correction_bias
        if self.use_grouped_topk:
            w, ids = ops.grouped_topk(router_logits, self.top_k, self.renormalize, self.num_expert_group,
                                      self.topk_group, self.scoring_func, bias, self.routed_scaling_factor)
        else:
            w, ids = ops.topk_gating(router_logits, self.top_k, self.renormalize, self.scoring_func, bias,
                                     self.routed_scaling_factor)
        if self.eplb:
            ids = self._to_physical(ids)
        return w, ids

    def _experts_sorted(self, a, a_scale, block_expert, total):
        qm = self.quant_method
        if qm is not None:
            return qm.apply_sorted(self, a, a_scale, block_expert, total)
        h = ops.gemm_grouped(a, self.w13_weight, block_expert, total, epi=1)
        return ops.gemm_grouped(h, self.w2_weight, block_expert, total)

    def _forward_sp(self, x: torch.Tensor, router_logits: torch.Tensor,
                    shared_out: Optional[torch.Tensor]) -> torch.Tensor:
        """Sequence-parallel MoE: every TP rank of a replica routes its own 1 / tp of the replica's tokens, rows travel
        once to the EP ranks that own their experts, partial sums come back, and the finished rows are all-gathered
        inside the replica - instead of every rank running its experts on all tokens and all-reducing ``[T, H]``.
        With several replicas the exchange spans all of them (DP attention + EP).  The reference's sequence-parallel
        MoE region (models/deepseek_v2.py:1273-1324) with its all2all managers
        (distributed/device_communicators/all2all.py:20-218)."""
        from ..parallel.all2all import AgRsAll2AllManager, NvlinkAll2AllManager, run_experts_a2a

        tpg, epg = ps.get_tp_group(), self.ep_group
        tp = tpg.world_size
        T, H = x.shape
        per = (T + tp - 1) // tp
        sizes = [max(0, min(per, T - r * per)) for r in range(tp)]
        lo, n = tpg.rank_in_group * per, sizes[tpg.rank_in_group]
        if n > 0:
            w, ids = self.route(router_logits[lo: lo + n])
        else:           # fewer tokens than ranks: this rank only serves its experts
            w = torch.empty(0, self.top_k, dtype=torch.float32, device=x.device)
            ids = torch.empty(0, self.top_k, dtype=torch.int32, device=x.device)
        mine_x = x[lo: lo + n].contiguous()
        qm = self.quant_method
        nvlink = self._nvlink_exchange(x)
        if nvlink:
            mgr = getattr(self, "_a2a", None)
            # replicas step with different token counts: the receive slots are sized once, for the largest step
            need = max(per, 64) if self.dp == 1 else max(64, -(-ps.max_tokens_per_step() // tp))
            if mgr is None or mgr.max_tokens < need:
                if mgr is not None:
                    mgr.close()
                mgr = NvlinkAll2AllManager(epg, need, H, self.top_k, self.num_physical, x.dtype, x.device,
                                           quant_fp8=bool(getattr(qm, "a2a_wire_fp8", False)))
                self._a2a = mgr
            mine = run_experts_a2a(mgr, mine_x, w, ids, self._experts_sorted)
        else:
            mgr = getattr(self, "_agrs", None)
            if mgr is None:
                mgr = self._agrs = AgRsAll2AllManager(epg)
            h_all, w_all, ids_all, _ = mgr.dispatch(mine_x, w, ids)
            if qm is not None:
                part = qm.apply(self, h_all, w_all, ids_all.to(torch.int32), None)
            else:
                part = fused_experts(h_all, self.w13_weight, self.w2_weight, w_all, ids_all.to(torch.int32),
                                     self.num_local, self.expert_map, None)
            mine = mgr.combine(part)
        y = tpg.all_gatherv(mine.contiguous(), sizes)
        if shared_out is not None:       # shared experts are tensor-parallel: their partial sums still need the reduction
            y = y + ps.tensor_model_parallel_all_reduce(shared_out)
        return y

    def _nvlink_exchange(self, x: torch.Tensor) -> bool:
        """Whether the token exchange runs over the NVLink dispatch / combine kernels: asked for by ``B200_MOE_A2A=1``
        or by ``use_sequence_parallel_moe`` with ``all2all_backend="fused_nvlink"``, on CUDA tensors whose rows the
        kernels take (hidden a multiple of 128; experts bf16 or a quantisation method with a sorted-rows entry)."""
        qm = self.quant_method
        want = bool(envs.B200_MOE_A2A) or (self._sp_config and ps.all2all_backend() == "fused_nvlink")
        return bool(want and x.is_cuda and x.shape[1] % 128 == 0 and (qm is None or hasattr(qm, "apply_sorted")))

    def sequence_parallel(self, x: torch.Tensor) -> bool:
        """Whether ``forward_reduced`` exchanges tokens (always with several replicas; opt-in inside one replica:
        ``B200_MOE_A2A=1`` for the NVLink kernels, or ``use_sequence_parallel_moe`` with either backend)."""
        if self.ep == 1:
            return False
        if self.dp > 1:
            return True
        if self._sp_config:
            return True
        return self._nvlink_exchange(x)

    def forward_reduced(self, x: torch.Tensor, router_logits: torch.Tensor,
                        shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The complete MoE output on every rank of the replica, whichever path computes it."""
        if self.sequence_parallel(x):
            return self._forward_sp(x, router_logits, shared_out)
        y = self.forward(x, router_logits, shared_out)
        if ps.tp_size() > 1 and not (self.reduce_results and self.ep > 1):
            y = ps.tensor_model_parallel_all_reduce(y)
        return y

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor,
                shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Local-filter path: this rank's experts on all of the replica's tokens (partial sums when ``ep > 1`` unless
        ``reduce_results``).  Not usable with several replicas, whose tokens differ."""
        assert self.dp == 1, "with data_parallel_size > 1 the experts need forward_reduced (tokens differ per replica)"
        if self.reduce_results and self.sequence_parallel(x):
            return self._forward_sp(x, router_logits, shared_out)
        w, ids = self.route(router_logits)

        def experts(xs, ws, idss, shared):
            if self.quant_method is not None:
                return self.quant_method.apply(self, xs, ws, idss, shared)
            return fused_experts(xs, self.w13_weight, self.w2_weight, ws, idss, self.num_local, self.expert_map, shared)

        chunk = int(envs.B200_FUSED_MOE_CHUNK_SIZE)
        T = x.shape[0]
        if chunk > 0 and T > chunk:
            # the expert-sorted copies of the rows ([T * top_k + padding, hidden] and [.., 2 * intermediate]) are the
            # layer's workspace: very long steps go through it in pieces
            y = torch.cat([experts(x[i: i + chunk], w[i: i + chunk], ids[i: i + chunk],
                                   None if shared_out is None else shared_out[i: i + chunk]) for i in range(0, T, chunk)])
        else:
            y = experts(x, w, ids, shared_out)
        if self.reduce_results and self.ep > 1:
            y = ps.tensor_model_parallel_all_reduce(y)
        return y


def reference_moe(x, w13, w2, topk_weights, topk_ids):
    """fp32 oracle on the interleaved-w13 layout."""
    gate, up = w13[:, 0::2], w13[:, 1::2]
    return ref.fused_experts(x, torch.cat([gate, up], dim=1), w2, topk_weights, topk_ids)
